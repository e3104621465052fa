// A recurrent mixer with a matrix state per head and a per-channel, data-dependent decay
// (RWKV-style time mixing):
//
//   mix_s[t] = x[t] + (x[t-1] - x[t]) * mu_s            s in {r, k, v, g, w};  x[-1] = 0
//   o[t]     = (S + diag(u) k[t] v[t]^T)^T r[t]         per head, S: [key channel, value channel]
//   S       <- diag(w[t]) S + k[t] v[t]^T               w[t] = exp(-exp(d[t] + w0))
//   y[t]     = o[t] / rms(o[t]) * norm * silu(g[t])     rms over a head's channels
//
// The state (S and the last x of the sequence) lives in 32-bit in the request's state slot and
// is carried from step to step; a fresh request starts from zeros.  Everything that enters the
// recurrence is 32-bit: decays, the bonus u, S, the sums.  Tokens are walked one after the other,
// each with the same order of additions, so the result does not depend on how a prompt was cut into steps.
#include "common.cuh"

namespace ff {

// One block per token: the five mixes.  The token in front is x[t-1] inside a portion and the
// state's saved row at its head (zeros for a fresh request).
template <typename T>
__global__ void wkv_shift_mix_kernel(const T* __restrict__ x, const float* __restrict__ mu /*[5,W]*/,
                                     const float* __restrict__ state, size_t state_stride, int prev_off,
                                     const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                                     const int* __restrict__ state_slots, const int* __restrict__ seq_fresh,
                                     T* __restrict__ mixes /*[5,T,W]*/, int Ttot, int W) {
    pdl_prologue();
    const int t = blockIdx.x;
    const int s = token_seq[t];
    const bool first = t == cu_q[s];
    const bool fresh = seq_fresh[s] != 0;
    const float* prev_state = state + (size_t)state_slots[s] * state_stride + prev_off;
    const T* xr = x + (size_t)t * W;
    const T* xp = x + (size_t)(t - 1) * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float cur = to_float(xr[i]);
        const float prev = first ? (fresh ? 0.f : prev_state[i]) : to_float(xp[i]);
        const float d = prev - cur;
#pragma unroll
        for (int m = 0; m < 5; ++m)
            mixes[((size_t)m * Ttot + t) * W + i] = from_float<T>(cur + d * mu[(size_t)m * W + i]);
    }
}

// tanh of a 32-bit matrix, into the type of the product that follows
template <typename TO>
__global__ void tanh_cast_kernel(const float* __restrict__ in, TO* __restrict__ out, size_t total) {
    pdl_prologue();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) out[idx] = from_float<TO>(tanhf(in[idx]));
}

constexpr int WKV_CHUNK = 8;     // tokens whose r, k, w are staged in shared memory at a time
// threads that share a column of S, each with a share of its key channels (a block has DIM * parts threads).
// Eight were tried up to head size 64 and were slower than four (1.30 against 1.11 ms for eight prompts of 2048).
constexpr int wkv_parts(int dim) { return 4; }

// One block per (sequence, head).  A column j of S (value channel j) is held by WKV_PARTS neighbouring
// threads, each with DIM / WKV_PARTS key channels in registers, so a token costs DIM / WKV_PARTS steps of the
// serial chain and two or three shuffles.  The bonus term's factors p_i = r_i u_i k_i are formed while a chunk is
// staged, so the inner loop has one multiply-add for it.
//   o_j = sum_i (r_i S_ij + p_i v_j);   S_ij <- w_i S_ij + k_i v_j
template <typename T, int DIM, int WKV_PARTS>
__global__ void __launch_bounds__(DIM * WKV_PARTS) wkv_scan_kernel(
    const T* __restrict__ rkvg /*[4,T,HD]*/, const float* __restrict__ dlog /*[T,HD]*/,
    const float* __restrict__ w0, const float* __restrict__ u, float* __restrict__ state, size_t state_stride,
    int prev_off, const T* __restrict__ x, int W, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, const int* __restrict__ seq_fresh, float* __restrict__ o /*[T,HD]*/,
    int Ttot, int heads, int dim) {
    pdl_prologue();
    constexpr int KP = DIM / WKV_PARTS;          // key channels a thread holds
    __shared__ __align__(16) float s_r[WKV_CHUNK][DIM], s_k[WKV_CHUNK][DIM], s_w[WKV_CHUNK][DIM], s_p[WKV_CHUNK][DIM];
    __shared__ float s_v[WKV_CHUNK][DIM];
    const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    // thread `part` of a column holds key channels 4 WKV_PARTS m + 4 part + e (m < KP / 4, e < 4): the parts of a
    // column then read neighbouring 16-byte pieces of shared memory, which lie in different banks
    const int j = tid / WKV_PARTS, part = tid % WKV_PARTS;
    auto chan = [&](int i) { return (i >> 2) * (4 * WKV_PARTS) + part * 4 + (i & 3); };
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    const int HD = heads * dim;
    const bool live = j < dim;
    float* st = state + (size_t)state_slots[s] * state_stride;
    // A head's state is kept in the slot as this kernel's threads hold it: element (register i, thread tid) at
    // i * blockDim + tid, DIM * DIM floats a head, so that loading and storing it is coalesced.  Only this kernel
    // reads it, and a layer always runs the same instantiation.
    float* S_g = st + (size_t)h * DIM * DIM;
    const bool fresh = seq_fresh[s] != 0;
    float S[KP];
#pragma unroll
    for (int i = 0; i < KP; ++i) S[i] = (live && chan(i) < dim && !fresh) ? S_g[i * (DIM * WKV_PARTS) + tid] : 0.f;
    // staging: thread c < dim takes channel c of every token of a chunk.  The next chunk's values are asked
    // for (into registers) before the current chunk is computed, so their latency hides behind the recurrence.
    const bool stager = tid < DIM, s_live = tid < dim;
    const float w0c = (stager && s_live) ? w0[h * dim + tid] : 0.f;
    const float uc = (stager && s_live) ? u[h * dim + tid] : 0.f;
    const T* r_in = rkvg;
    const T* k_in = rkvg + (size_t)Ttot * HD;
    const T* v_in = rkvg + (size_t)2 * Ttot * HD;
    T rn[WKV_CHUNK], kn[WKV_CHUNK], vn[WKV_CHUNK];
    float dn[WKV_CHUNK];
    auto fetch = [&](int c0) {
#pragma unroll
        for (int c = 0; c < WKV_CHUNK; ++c) {
            const bool in = stager && s_live && c0 + c < t1;
            const size_t at = in ? (size_t)(c0 + c) * HD + h * dim + tid : 0;
            rn[c] = in ? r_in[at] : from_float<T>(0.f);
            kn[c] = in ? k_in[at] : from_float<T>(0.f);
            vn[c] = in ? v_in[at] : from_float<T>(0.f);
            dn[c] = in ? dlog[at] : 0.f;
        }
    };
    fetch(t0);
    for (int c0 = t0; c0 < t1; c0 += WKV_CHUNK) {
        const int n = min(WKV_CHUNK, t1 - c0);
        __syncthreads();
        if (stager) {
#pragma unroll
            for (int c = 0; c < WKV_CHUNK; ++c) {
                const bool in = s_live && c < n;
                const float rv = to_float(rn[c]), kv = to_float(kn[c]);
                s_r[c][tid] = rv;
                s_k[c][tid] = kv;
                s_v[c][tid] = to_float(vn[c]);
                s_w[c][tid] = in ? expf(-expf(dn[c] + w0c)) : 1.f;
                s_p[c][tid] = rv * uc * kv;
            }
        }
        __syncthreads();
        if (c0 + WKV_CHUNK < t1) fetch(c0 + WKV_CHUNK);
        // Four partial sums shorten the chain inside a token.  (Computing all eight places of a chunk without a
        // branch, the places past the portion's end staged as values that leave S alone, was no faster for
        // prompts, 1.07 against 1.11 ms, and made a step of single tokens half again as slow.)  What bounds a
        // token is the shared-memory pipe: every thread reads r, k, w and p of its sixteen channels.
#pragma unroll
        for (int c = 0; c < WKV_CHUNK; ++c) {
            if (c < n) {
                const float vj = s_v[c][j];
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int i = 0; i < KP; i += 4) {
                    const int at = i * WKV_PARTS + part * 4;      // = chan(i), i a multiple of 4
                    const float4 r4 = *reinterpret_cast<const float4*>(&s_r[c][at]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&s_k[c][at]);
                    const float4 w4 = *reinterpret_cast<const float4*>(&s_w[c][at]);
                    const float4 p4 = *reinterpret_cast<const float4*>(&s_p[c][at]);
                    a0 += r4.x * S[i] + p4.x * vj;     S[i]     = w4.x * S[i]     + k4.x * vj;
                    a1 += r4.y * S[i + 1] + p4.y * vj; S[i + 1] = w4.y * S[i + 1] + k4.y * vj;
                    a2 += r4.z * S[i + 2] + p4.z * vj; S[i + 2] = w4.z * S[i + 2] + k4.z * vj;
                    a3 += r4.w * S[i + 3] + p4.w * vj; S[i + 3] = w4.w * S[i + 3] + k4.w * vj;
                }
                float acc = (a0 + a1) + (a2 + a3);
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                if (WKV_PARTS == 8) acc += __shfl_xor_sync(0xffffffffu, acc, 4);
                if (live && part == 0) o[(size_t)(c0 + c) * HD + h * dim + j] = acc;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < KP; ++i) S_g[i * (DIM * WKV_PARTS) + tid] = (live && chan(i) < dim) ? S[i] : 0.f;
    // the sequence's last input row, for the first token of its next step
    if (h == 0 && t1 > t0) {
        const T* last = x + (size_t)(t1 - 1) * W;
        for (int i = tid; i < W; i += DIM * WKV_PARTS) st[prev_off + i] = to_float(last[i]);
        static_assert(WKV_PARTS == 4 || WKV_PARTS == 8, "the sum over a column's threads is two or three shuffles");
    }
}

// One warp per (token, head): y = o / rms(o) * norm * silu(g)
template <typename T>
__global__ void wkv_out_kernel(const float* __restrict__ o, const T* __restrict__ g, const float* __restrict__ norm,
                               float eps, T* __restrict__ y, int Ttot, int heads, int dim) {
    pdl_prologue();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= Ttot * heads) return;
    const int t = warp / heads, h = warp - t * heads;
    const size_t base = (size_t)t * heads * dim + (size_t)h * dim;
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) { const float v = o[base + i]; ss += v * v; }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    for (int i = lane; i < dim; i += 32) {
        const float gv = to_float(g[base + i]);
        y[base + i] = from_float<T>(o[base + i] * inv * norm[h * dim + i] * (gv / (1.0f + expf(-gv))));
    }
}

}  // namespace ff

using namespace ff;

FF_EXPORT int ff_wkv_shift_mix(const void* x, int dtype, const float* mu, const float* state, long long state_stride,
                               int prev_off, const int* token_seq, const int* cu_q, const int* state_slots,
                               const int* seq_fresh, void* mixes, int T, int W, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int threads = W >= 1024 ? 256 : 128;
    if (dtype == 0)
        FF_LAUNCH((wkv_shift_mix_kernel<float>), T, threads, 0, stream, (const float*)x, mu, state, (size_t)state_stride,
                  prev_off, token_seq, cu_q, state_slots, seq_fresh, (float*)mixes, T, W);
    else if (dtype == 1)
        FF_LAUNCH((wkv_shift_mix_kernel<bf16>), T, threads, 0, stream, (const bf16*)x, mu, state, (size_t)state_stride,
                  prev_off, token_seq, cu_q, state_slots, seq_fresh, (bf16*)mixes, T, W);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_tanh_cast(const float* in, void* out, int out_dtype, long long total, cudaStream_t stream) {
    if (total <= 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == 0) FF_LAUNCH((tanh_cast_kernel<float>), blocks, 256, 0, stream, in, (float*)out, (size_t)total);
    else if (out_dtype == 1) FF_LAUNCH((tanh_cast_kernel<bf16>), blocks, 256, 0, stream, in, (bf16*)out, (size_t)total);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int wkv_scan_launch(const void* rkvg, const float* dlog, const float* w0, const float* u, float* state,
                           long long state_stride, int prev_off, const void* x, int W, const int* cu_q,
                           const int* state_slots, const int* seq_fresh, float* o, int Ttot, int n_seqs, int heads,
                           int dim, cudaStream_t stream) {
    dim3 grid(n_seqs, heads);
#define FF_WKV(D)                                                                                                  \
    FF_LAUNCH((wkv_scan_kernel<T, D, wkv_parts(D)>), grid, D * wkv_parts(D), 0, stream, (const T*)rkvg, dlog, w0, u, state, (size_t)state_stride, \
              prev_off, (const T*)x, W, cu_q, state_slots, seq_fresh, o, Ttot, heads, dim)
    if (dim <= 32) FF_WKV(32);
    else if (dim <= 64) FF_WKV(64);
    else if (dim <= 128) FF_WKV(128);
    else return FF_ERR_UNSUPPORTED;
#undef FF_WKV
    FF_LAUNCH_CHECK();
    return 0;
}

// the head size the recurrence kernel is instantiated for (its state keeps that many squared floats a head)
FF_EXPORT int ff_wkv_state_dim(int dim) { return dim <= 32 ? 32 : (dim <= 64 ? 64 : (dim <= 128 ? 128 : -1)); }

FF_EXPORT int ff_wkv_scan(const void* rkvg, int dtype, const float* dlog, const float* w0, const float* u, float* state,
                          long long state_stride, int prev_off, const void* x, int W, const int* cu_q,
                          const int* state_slots, const int* seq_fresh, float* o, int Ttot, int n_seqs, int heads,
                          int dim, cudaStream_t stream) {
    if (Ttot <= 0 || n_seqs <= 0) return 0;
    if (dtype == 0)
        return wkv_scan_launch<float>(rkvg, dlog, w0, u, state, state_stride, prev_off, x, W, cu_q, state_slots,
                                      seq_fresh, o, Ttot, n_seqs, heads, dim, stream);
    if (dtype == 1)
        return wkv_scan_launch<bf16>(rkvg, dlog, w0, u, state, state_stride, prev_off, x, W, cu_q, state_slots,
                                     seq_fresh, o, Ttot, n_seqs, heads, dim, stream);
    return FF_ERR_BAD_ARG;
}

FF_EXPORT int ff_wkv_out(const float* o, const void* g, int dtype, const float* norm, float eps, void* y, int T,
                         int heads, int dim, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long warps = (long long)T * heads;
    const unsigned blocks = (unsigned)((warps + 3) / 4);
    if (dtype == 0)
        FF_LAUNCH((wkv_out_kernel<float>), blocks, 128, 0, stream, o, (const float*)g, norm, eps, (float*)y, T, heads, dim);
    else if (dtype == 1)
        FF_LAUNCH((wkv_out_kernel<bf16>), blocks, 128, 0, stream, o, (const bf16*)g, norm, eps, (bf16*)y, T, heads, dim);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
