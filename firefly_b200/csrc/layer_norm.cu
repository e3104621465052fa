// Layer normalisation with weight and bias over the 32-bit residual stream, and the
// small row kernels that a looped range of layers needs at the head of a pass.
//
//   residual[s,:] (+= delta_scale * delta[s,:]);  v = residual[s,:]
//   out[r,:] = (v - mean(v)) / sqrt(mean((v - mean)^2) + eps) * w + b
//
// Statistics in 32-bit, two passes over the row held in shared memory (the variance is
// the mean of the squared deviations, not E[v^2] - mean^2).  s = row_idx ? row_idx[r] : r;
// with row_idx the residual is not written back.
#include "common.cuh"

namespace ff {

template <typename TD, typename TO>
__global__ void add_layer_norm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, float delta_scale,
                                      const int* __restrict__ row_idx, const float* __restrict__ w,
                                      const float* __restrict__ b, float eps, TO* __restrict__ out, int H,
                                      int write_residual) {
    pdl_prologue();
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src = row_idx ? row_idx[r] : r;
    float* res = residual + (size_t)src * H;
    const TD* dl = delta ? delta + (size_t)src * H : nullptr;
    float sum = 0.f;
    if ((H & 3) == 0) {       // four elements a thread and step
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(res + i);
            if (dl) {
                v.x += delta_scale * to_float(dl[i]);     v.y += delta_scale * to_float(dl[i + 1]);
                v.z += delta_scale * to_float(dl[i + 2]); v.w += delta_scale * to_float(dl[i + 3]);
                if (write_residual) *reinterpret_cast<float4*>(res + i) = v;
            }
            *reinterpret_cast<float4*>(row + i) = v;
            sum += (v.x + v.y) + (v.z + v.w);
        }
    } else
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = res[i];
        if (dl) {
            v += delta_scale * to_float(dl[i]);
            if (write_residual) res[i] = v;
        }
        row[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)H;
    float sq = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = row[i] - mean;
        sq += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)H + eps);
    TO* o = out + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_float<TO>((row[i] - mean) * inv * w[i] + (b ? b[i] : 0.f));
}

// out[t, 0:H] = a[t,:], out[t, H:2H] = b[t,:]  (two 32-bit streams side by side, in the product's type)
template <typename TO>
__global__ void concat_cast_kernel(const float* __restrict__ a, const float* __restrict__ b, TO* __restrict__ out,
                                   int H, size_t total) {
    pdl_prologue();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / (2 * H);
    const int i = (int)(idx - t * 2 * H);
    out[idx] = from_float<TO>(i < H ? a[t * H + i] : b[t * H + (i - H)]);
}

// x[t,:] += scale * v[:]
__global__ void add_row_vector_kernel(float* __restrict__ x, const float* __restrict__ v, float scale, int H,
                                      size_t total) {
    pdl_prologue();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    x[idx] += scale * v[idx % H];
}

}  // namespace ff

using namespace ff;

FF_EXPORT int ff_add_layer_norm(float* residual, const void* delta, int delta_dtype, float delta_scale,
                                const int* row_idx, const float* w, const float* b, float eps, void* out,
                                int out_dtype, int rows, int H, int write_residual, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0) return FF_ERR_BAD_ARG;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return FF_ERR_UNSUPPORTED;
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
#define FF_LN(TD, TO)                                                                                        \
    do {                                                                                                     \
        if (smem > 48 * 1024) FF_SMEM_LIMIT((add_layer_norm_kernel<TD, TO>), smem);                          \
        FF_LAUNCH((add_layer_norm_kernel<TD, TO>), rows, threads, smem, stream, residual, (const TD*)delta,  \
                  delta_scale, row_idx, w, b, eps, (TO*)out, H, write_residual);                             \
    } while (0)
    if (delta_dtype == 0 && out_dtype == 0) FF_LN(float, float);
    else if (delta_dtype == 0 && out_dtype == 1) FF_LN(float, bf16);
    else if (delta_dtype == 1 && out_dtype == 0) FF_LN(bf16, float);
    else if (delta_dtype == 1 && out_dtype == 1) FF_LN(bf16, bf16);
    else return FF_ERR_BAD_ARG;
#undef FF_LN
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_concat_cast(const float* a, const float* b, void* out, int out_dtype, int T, int H,
                             cudaStream_t stream) {
    const size_t total = (size_t)T * 2 * H;
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (out_dtype == 0) FF_LAUNCH((concat_cast_kernel<float>), blocks, 256, 0, stream, a, b, (float*)out, H, total);
    else if (out_dtype == 1) FF_LAUNCH((concat_cast_kernel<bf16>), blocks, 256, 0, stream, a, b, (bf16*)out, H, total);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_add_row_vector(float* x, const float* v, float scale, int T, int H, cudaStream_t stream) {
    const size_t total = (size_t)T * H;
    if (total == 0) return 0;
    FF_LAUNCH(add_row_vector_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, x, v, scale, H, total);
    FF_LAUNCH_CHECK();
    return 0;
}
