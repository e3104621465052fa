// Recurrent mixers whose state decays by one scalar per head and token:
//
//   S_t = a_t S_(t-1) + b_t k_t v_t^T        S: [key channel, value channel] per head, 32-bit, starts at 0
//   o_t = S_t^T q_t  (+ D v_t)
//
// Two designs use it.  A state-space mixer (Mamba-2 style): k = B_t and q = C_t (shared by the heads of a
// group), v = x_t, step = softplus(raw_t + bias), a_t = exp(-exp(A_log) step), b_t = step, with a skip
// term D x_t; its inputs x, B, C come out of a short causal convolution per channel with SiLU
// (`causal_conv_silu_kernel`), whose last taps-1 inputs are part of the request's state.  And linear
// attention with a constant decay per head: a = decay_h, b = 1, q, k, v = SiLU of three projections.
//
// The state lives in the request's state slot in 32-bit and is carried from step to step; a fresh request
// starts from zeros.  Decays, steps, S and every sum are 32-bit.  A sequence's tokens are walked in order
// with the same order of additions however the prompt was cut into steps.
#include "common.cuh"

namespace ff {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// ----------------------------------------------------------------------------- convolution --
// out[t, c] = silu(bias[c] + sum_j w[c, j] * in[t - (taps-1) + j, c]); inputs in front of the portion come
// from the state slot (`conv_off`: [(taps-1), C] floats, oldest first; zeros for a fresh request).
template <typename T>
__global__ void causal_conv_silu_kernel(const T* in, int in_stride, int in_off,
                                        const float* __restrict__ w /*[C,taps]*/, const float* __restrict__ bias,
                                        const float* state, size_t state_stride, int conv_off,
                                        const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                                        const int* __restrict__ state_slots, const int* __restrict__ seq_fresh,
                                        T* __restrict__ out /*[T,C]*/, int C, int taps) {
    pdl_prologue();
    in = pdl_fresh(in);
    state = pdl_fresh(state);
    const int t = blockIdx.x;
    const int s = token_seq[t];
    const int t0 = cu_q[s];
    const bool fresh = seq_fresh[s] != 0;
    const float* st = state + (size_t)state_slots[s] * state_stride + conv_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc = bias[c];
        for (int j = 0; j < taps; ++j) {
            const int tt = t - (taps - 1) + j;
            float v;
            if (tt >= t0) v = to_float(in[(size_t)tt * in_stride + in_off + c]);
            else {
                const int r = (taps - 1) + (tt - t0);       // row of the saved inputs: 0 oldest
                v = fresh ? 0.f : st[(size_t)r * C + c];
            }
            acc += w[(size_t)c * taps + j] * v;
        }
        out[(size_t)t * C + c] = from_float<T>(silu_f(acc));
    }
}

// The last taps-1 inputs of every sequence, for its next step.  One thread per (sequence, channel) reads what
// it needs of the old rows before it writes.
template <typename T>
__global__ void conv_state_update_kernel(const T* in, int in_stride, int in_off, float* __restrict__ state,
                                         size_t state_stride, int conv_off, const int* __restrict__ cu_q,
                                         const int* __restrict__ state_slots, const int* __restrict__ seq_fresh,
                                         int C, int taps) {
    pdl_prologue();
    in = pdl_fresh(in);
    constexpr int MAX_KEEP = 15;
    const int s = blockIdx.x;
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    const int keep = taps - 1, n = t1 - t0;
    if (n <= 0) return;
    const bool fresh = seq_fresh[s] != 0;
    float* st = state + (size_t)state_slots[s] * state_stride + conv_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float nv[MAX_KEEP];
#pragma unroll
        for (int r = 0; r < MAX_KEEP; ++r) {
            if (r < keep) {
                const int tt = t1 - keep + r;
                if (tt >= t0) nv[r] = to_float(in[(size_t)tt * in_stride + in_off + c]);
                else nv[r] = fresh ? 0.f : st[(size_t)(keep + (tt - t0)) * C + c];
            }
        }
#pragma unroll
        for (int r = 0; r < MAX_KEEP; ++r)
            if (r < keep) st[(size_t)r * C + c] = nv[r];
    }
}

// ----------------------------------------------------------------------------- the recurrence --
struct ScanArgs {
    const void* q; int q_stride, q_off;          // [T, ...] key-sized rows per group: q_off + group * N + i
    const void* k; int k_stride, k_off;
    const void* v; int v_stride, v_off;          // value rows per head: v_off + h * V + j
    int heads_per_group;                         // heads that share one q/k row (1: a row per head)
    int act;                                     // 1: q, k, v pass SiLU as they are read
    const float* decay;                          // [heads] constant a (mode 0)
    const void* step; int step_stride, step_off; // mode 1: raw step per (token, head)
    const float* step_bias; const float* a_log; const float* skip;   // [heads] each (mode 1; skip may be null)
    int mode;
};

constexpr int SCAN_CHUNK = 8;

// One block per (sequence, head).  Value channel j is held by PARTS neighbouring threads, each with NP / PARTS key
// channels of column j in registers.  NP: the key size rounded up to the instantiation.
template <typename T, int NP, int PARTS>
__global__ void __launch_bounds__(512) scalar_decay_scan_kernel(
    ScanArgs A, float* __restrict__ state, size_t state_stride, int state_off, const int* __restrict__ cu_q,
    const int* __restrict__ state_slots, const int* __restrict__ seq_fresh, float* __restrict__ o /*[T, heads*V]*/,
    int heads, int N, int V) {
    pdl_prologue();
    constexpr int KP = NP / PARTS;
    __shared__ __align__(16) float s_q[SCAN_CHUNK][NP], s_k[SCAN_CHUNK][NP];
    __shared__ float s_v[SCAN_CHUNK][128];
    __shared__ float s_a[SCAN_CHUNK], s_d[SCAN_CHUNK];
    const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, nthr = blockDim.x;
    const int j = tid / PARTS, part = tid % PARTS;
    const int t0 = cu_q[s], t1 = cu_q[s + 1];
    const bool live = j < V;
    const bool fresh = seq_fresh[s] != 0;
    // a head's state is kept as this kernel's threads hold it: register i of thread tid at i * threads + tid
    float* S_g = state + (size_t)state_slots[s] * state_stride + state_off + (size_t)h * KP * nthr;
    float S[KP];
#pragma unroll
    for (int i = 0; i < KP; ++i) S[i] = fresh ? 0.f : S_g[(size_t)i * nthr + tid];
    const int group = h / A.heads_per_group;
    const T* qp = pdl_fresh((const T*)A.q) + A.q_off + (size_t)group * N;
    const T* kp = pdl_fresh((const T*)A.k) + A.k_off + (size_t)group * N;
    const T* vp = pdl_fresh((const T*)A.v) + A.v_off + (size_t)h * V;
    const T* stepp = pdl_fresh((const T*)A.step);
    float a_const = 1.f, rate = 0.f, sbias = 0.f, skip = 0.f;
    if (A.mode == 0) a_const = A.decay[h];
    else { rate = expf(A.a_log[h]); sbias = A.step_bias[h]; skip = A.skip ? A.skip[h] : 0.f; }
    for (int c0 = t0; c0 < t1; c0 += SCAN_CHUNK) {
        const int n = min(SCAN_CHUNK, t1 - c0);
        __syncthreads();
        // staging: the chunk's q, b*k, v and decays in 32-bit
        if (tid < SCAN_CHUNK) {
            float a = a_const, b = 1.f;
            if (A.mode == 1 && tid < n) {
                const float raw = to_float(stepp[(size_t)(c0 + tid) * A.step_stride + A.step_off + h]);
                const float dt = softplus_f(raw + sbias);
                a = expf(-rate * dt);
                b = dt;
            }
            s_a[tid] = a;
            s_d[tid] = b;
        }
        __syncthreads();
        for (int idx = tid; idx < SCAN_CHUNK * NP; idx += nthr) {
            const int c = idx / NP, i = idx - c * NP;
            float qv = 0.f, kv = 0.f;
            if (c < n && i < N) {
                qv = to_float(qp[(size_t)(c0 + c) * A.q_stride + i]);
                kv = to_float(kp[(size_t)(c0 + c) * A.k_stride + i]);
                if (A.act) { qv = silu_f(qv); kv = silu_f(kv); }
                kv *= s_d[c];
            }
            s_q[c][i] = qv;
            s_k[c][i] = kv;
        }
        for (int idx = tid; idx < SCAN_CHUNK * V; idx += nthr) {
            const int c = idx / V, jj = idx - c * V;
            float vv = 0.f;
            if (c < n) {
                vv = to_float(vp[(size_t)(c0 + c) * A.v_stride + jj]);
                if (A.act) vv = silu_f(vv);
            }
            s_v[c][jj] = vv;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < SCAN_CHUNK; ++c) {
            if (c < n) {
                const float vj = live ? s_v[c][j] : 0.f;
                const float a = s_a[c];
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                for (int i = 0; i < KP; i += 4) {
                    // thread `part` holds key channels 4 PARTS m + 4 part + e (m = i / 4, e < 4)
                    const int at = i * PARTS + part * 4;
                    const float4 q4 = *reinterpret_cast<const float4*>(&s_q[c][at]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&s_k[c][at]);
                    S[i]     = a * S[i]     + k4.x * vj;  a0 += q4.x * S[i];
                    S[i + 1] = a * S[i + 1] + k4.y * vj;  a1 += q4.y * S[i + 1];
                    S[i + 2] = a * S[i + 2] + k4.z * vj;  a2 += q4.z * S[i + 2];
                    S[i + 3] = a * S[i + 3] + k4.w * vj;  a3 += q4.w * S[i + 3];
                }
                float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
                for (int off = 1; off < PARTS; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
                if (live && part == 0) o[(size_t)(c0 + c) * heads * V + (size_t)h * V + j] = acc + skip * vj;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < KP; ++i) S_g[(size_t)i * nthr + tid] = S[i];
}

// ----------------------------------------------------------------------------- gate and norm --
// One block per (token, part).  order 0: y = rms(o * silu(z)) * w  (the gate in front of the norm, norm over
// each of `parts` equal parts);  order 1: y = rms(o) * w * sigmoid(z)  (the gate behind it).
template <typename T>
__global__ void gated_rms_norm_kernel(const float* o, const T* z, int z_stride, int z_off,
                                      const float* __restrict__ w, float eps, T* __restrict__ y, int width, int parts,
                                      int order) {
    pdl_prologue();
    o = pdl_fresh(o);
    z = pdl_fresh(z);
    __shared__ float scratch[32];
    const int t = blockIdx.x, g = blockIdx.y;
    const int per = width / parts;
    const float* orow = o + (size_t)t * width + (size_t)g * per;
    const T* zrow = z + (size_t)t * z_stride + z_off + (size_t)g * per;
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        float v = orow[i];
        if (order == 0) v *= silu_f(to_float(zrow[i]));
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)per + eps);
    T* yrow = y + (size_t)t * width + (size_t)g * per;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const float zv = to_float(zrow[i]);
        float v = orow[i];
        if (order == 0) v = v * silu_f(zv) * inv * w[g * per + i];
        else v = v * inv * w[g * per + i] / (1.0f + expf(-zv));
        yrow[i] = from_float<T>(v);
    }
}

}  // namespace ff

using namespace ff;

FF_EXPORT int ff_causal_conv_silu(const void* in, int dtype, int in_stride, int in_off, const float* w, const float* bias,
                                  float* state, long long state_stride, int conv_off, const int* token_seq,
                                  const int* cu_q, const int* state_slots, const int* seq_fresh, void* out, int T,
                                  int n_seqs, int C, int taps, cudaStream_t stream) {
    if (T <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > 16) return FF_ERR_UNSUPPORTED;
    const int cy = min(64, (C + 255) / 256);
    if (dtype == 0) {
        FF_LAUNCH((causal_conv_silu_kernel<float>), dim3(T, cy), 256, 0, stream, (const float*)in, in_stride, in_off, w, bias,
                  (const float*)state, (size_t)state_stride, conv_off, token_seq, cu_q, state_slots, seq_fresh, (float*)out, C, taps);
        if (taps > 1)
            FF_LAUNCH((conv_state_update_kernel<float>), dim3(n_seqs, cy), 256, 0, stream, (const float*)in, in_stride, in_off,
                      state, (size_t)state_stride, conv_off, cu_q, state_slots, seq_fresh, C, taps);
    } else if (dtype == 1) {
        FF_LAUNCH((causal_conv_silu_kernel<bf16>), dim3(T, cy), 256, 0, stream, (const bf16*)in, in_stride, in_off, w, bias,
                  (const float*)state, (size_t)state_stride, conv_off, token_seq, cu_q, state_slots, seq_fresh, (bf16*)out, C, taps);
        if (taps > 1)
            FF_LAUNCH((conv_state_update_kernel<bf16>), dim3(n_seqs, cy), 256, 0, stream, (const bf16*)in, in_stride, in_off,
                      state, (size_t)state_stride, conv_off, cu_q, state_slots, seq_fresh, C, taps);
    } else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

// key size the recurrence is instantiated for, and threads of a block (a column's threads times the value size,
// rounded up to whole warps); -1: not supported
FF_EXPORT int ff_scan_key_pad(int N) { return N <= 16 ? 16 : (N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : -1))); }
FF_EXPORT int ff_scan_threads(int V) { return V <= 0 || V > 128 ? -1 : ((V * 4 + 31) / 32) * 32; }

template <typename T>
static int scan_launch(const ScanArgs& A, float* state, long long state_stride, int state_off, const int* cu_q,
                       const int* state_slots, const int* seq_fresh, float* o, int n_seqs, int heads, int N, int V,
                       cudaStream_t stream) {
    const int threads = ff_scan_threads(V);
    if (threads < 0) return FF_ERR_UNSUPPORTED;
    dim3 grid(n_seqs, heads);
#define FF_SCAN(NP)                                                                                              \
    FF_LAUNCH((scalar_decay_scan_kernel<T, NP, 4>), grid, threads, 0, stream, A, state, (size_t)state_stride, state_off, \
              cu_q, state_slots, seq_fresh, o, heads, N, V)
    switch (ff_scan_key_pad(N)) {
        case 16: FF_SCAN(16); break;
        case 32: FF_SCAN(32); break;
        case 64: FF_SCAN(64); break;
        case 128: FF_SCAN(128); break;
        default: return FF_ERR_UNSUPPORTED;
    }
#undef FF_SCAN
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_scalar_decay_scan(const void* q, int q_stride, int q_off, const void* k, int k_stride, int k_off,
                                   const void* v, int v_stride, int v_off, int dtype, int heads_per_group, int act,
                                   int mode, const float* decay, const void* step, int step_stride, int step_off,
                                   const float* step_bias, const float* a_log, const float* skip, float* state,
                                   long long state_stride, int state_off, const int* cu_q, const int* state_slots,
                                   const int* seq_fresh, float* o, int T, int n_seqs, int heads, int N, int V,
                                   cudaStream_t stream) {
    if (T <= 0 || n_seqs <= 0) return 0;
    if (heads_per_group <= 0 || (mode != 0 && mode != 1)) return FF_ERR_BAD_ARG;
    ScanArgs A{q, q_stride, q_off, k, k_stride, k_off, v, v_stride, v_off, heads_per_group, act, decay,
               step, step_stride, step_off, step_bias, a_log, skip, mode};
    if (dtype == 0)
        return scan_launch<float>(A, state, state_stride, state_off, cu_q, state_slots, seq_fresh, o, n_seqs, heads, N, V, stream);
    if (dtype == 1)
        return scan_launch<bf16>(A, state, state_stride, state_off, cu_q, state_slots, seq_fresh, o, n_seqs, heads, N, V, stream);
    return FF_ERR_BAD_ARG;
}

FF_EXPORT int ff_gated_rms_norm(const float* o, const void* z, int dtype, int z_stride, int z_off, const float* w,
                                float eps, void* y, int T, int width, int parts, int order, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (parts <= 0 || width % parts || (order != 0 && order != 1)) return FF_ERR_BAD_ARG;
    const int per = width / parts;
    const int threads = per >= 1024 ? 256 : (per >= 256 ? 128 : 64);
    if (dtype == 0)
        FF_LAUNCH((gated_rms_norm_kernel<float>), dim3(T, parts), threads, 0, stream, o, (const float*)z, z_stride, z_off, w, eps,
                  (float*)y, width, parts, order);
    else if (dtype == 1)
        FF_LAUNCH((gated_rms_norm_kernel<bf16>), dim3(T, parts), threads, 0, stream, o, (const bf16*)z, z_stride, z_off, w, eps,
                  (bf16*)y, width, parts, order);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}
