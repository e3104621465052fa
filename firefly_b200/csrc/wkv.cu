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
// so the result does not depend on how a prompt was cut into steps.
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

// One block per (sequence, head); thread j owns value channel j and column j of S in registers.
template <typename T, int DIM>
__global__ void __launch_bounds__(DIM) wkv_scan_kernel(
    const T* __restrict__ rkvg /*[4,T,HD]*/, const float* __restrict__ dlog /*[T,HD]*/,
    const float* __restrict__ w0, const float* __restrict__ u, float* __restrict__ state, size_t state_stride,
    int prev_off, const T* __restrict__ x, int W, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, const int* __restrict__ seq_fresh, float* __restrict__ o /*[T,HD]*/,
    int Ttot, int heads, int dim) {
    pdl_prologue();
    __shared__ float s_r[WKV_CHUNK][DIM], s_k[WKV_CHUNK][DIM], s_w[WKV_CHUNK][DIM], s_u[DIM];
    const int s = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    const int HD = heads * dim;
    const bool live = j < dim;
    float* st = state + (size_t)state_slots[s] * state_stride;
    float* S_g = st + (size_t)h * dim * dim;
    const bool fresh = seq_fresh[s] != 0;
    float S[DIM];
#pragma unroll
    for (int i = 0; i < DIM; ++i) S[i] = (live && i < dim && !fresh) ? S_g[(size_t)i * dim + j] : 0.f;
    s_u[j] = live ? u[h * dim + j] : 0.f;
    const float w0j = live ? w0[h * dim + j] : 0.f;
    const T* r_in = rkvg;
    const T* k_in = rkvg + (size_t)Ttot * HD;
    const T* v_in = rkvg + (size_t)2 * Ttot * HD;
    for (int c0 = t0; c0 < t1; c0 += WKV_CHUNK) {
        const int n = min(WKV_CHUNK, t1 - c0);
        float v[WKV_CHUNK];
        __syncthreads();
#pragma unroll
        for (int c = 0; c < WKV_CHUNK; ++c) {
            if (c < n && live) {
                const size_t at = (size_t)(c0 + c) * HD + h * dim + j;
                s_r[c][j] = to_float(r_in[at]);
                s_k[c][j] = to_float(k_in[at]);
                s_w[c][j] = expf(-expf(dlog[at] + w0j));
                v[c] = to_float(v_in[at]);
            } else {
                s_r[c][j] = 0.f; s_k[c][j] = 0.f; s_w[c][j] = 1.f;
                v[c] = 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < WKV_CHUNK; ++c) {
            if (c < n) {
                const float vj = v[c];
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < DIM; ++i) {
                    const float kv = s_k[c][i] * vj;
                    acc += s_r[c][i] * (S[i] + s_u[i] * kv);
                    S[i] = s_w[c][i] * S[i] + kv;
                }
                if (live) o[(size_t)(c0 + c) * HD + h * dim + j] = acc;
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DIM; ++i)
            if (i < dim) S_g[(size_t)i * dim + j] = S[i];
    }
    // the sequence's last input row, for the first token of its next step
    if (h == 0 && t1 > t0) {
        const T* last = x + (size_t)(t1 - 1) * W;
        for (int i = j; i < W; i += DIM) st[prev_off + i] = to_float(last[i]);
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
    FF_LAUNCH((wkv_scan_kernel<T, D>), grid, D, 0, stream, (const T*)rkvg, dlog, w0, u, state, (size_t)state_stride, \
              prev_off, (const T*)x, W, cu_q, state_slots, seq_fresh, o, Ttot, heads, dim)
    if (dim <= 32) FF_WKV(32);
    else if (dim <= 64) FF_WKV(64);
    else if (dim <= 128) FF_WKV(128);
    else return FF_ERR_UNSUPPORTED;
#undef FF_WKV
    FF_LAUNCH_CHECK();
    return 0;
}

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
