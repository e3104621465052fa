// Routed experts: the router's choice, the plan that sorts a step's tokens by expert, the
// grouped products over the experts' stacked matrices, and the weighted sum back into the
// 32-bit residual.  Nothing here is read by the host: counts, offsets and the list of row
// tiles stay on the device, and the grouped products are launched for the largest number of
// tiles a step of that many tokens can have (blocks past the real count leave at once), so a
// step with routed experts can be captured into a CUDA graph.
//
//   s = softmax(z) over all experts (32-bit).  Experts form `groups` equal groups of
//   neighbours; a group's score is its largest s; only experts of the `keep` best groups may
//   be chosen; of those the `top` with the largest s are; weights = s / (sum of chosen s + 1e-20).
//   expert(h) = W_down (g * sigmoid(1.702 g) * (u + 1)),  g = min(W_gate h, limit),
//   u = clamp(W_up h, -limit, limit).
//
// A row of a grouped product is one (token, choice) pair; its result is a plain dot product
// per output in a fixed order over K, so it does not depend on which other rows share its tile.
#include "common.cuh"
#include <math_constants.h>

namespace ff {

constexpr int MOE_BM = 64, MOE_BN = 64, MOE_BK = 16;

// act 1: silu(g) * u, no clamps.  act 0: the clamped form below.
__device__ __forceinline__ float clamped_glu(float g, float u, float limit, int act = 0) {
    if (act == 1) return g / (1.0f + expf(-g)) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
}

// (value, index) arg-max over a warp; the lowest index wins ties
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

// One warp per token.  score 0: s = softmax(z) over all experts; 1: s = sigmoid(z).  The choice uses
// c = s + correction (correction may be null); a group's score is its largest c (group_score 0) or the sum of
// its two largest (1); experts of closed groups count as minus infinity (c may be negative); the weights are the
// chosen experts' s, divided by their sum (+ 1e-20) when `renorm`.  Ties go to the lowest index.
__global__ void moe_route_kernel(const float* z, const float* __restrict__ correction, int T, int E, int top,
                                 int groups, int keep, int score, int group_score, int renorm,
                                 int* __restrict__ ids, float* __restrict__ wts) {
    pdl_prologue();
    z = pdl_fresh(z);
    extern __shared__ float sh[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* s = sh + (size_t)warp * (2 * E + 2 * groups);
    float* a = s + E;              // choice scores; minus infinity when closed or taken
    float* gs = a + E;
    float* g_open = gs + groups;
    const float* zr = z + (size_t)t * E;
    if (score == 0) {
        float mx = -CUDART_INF_F;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, zr[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float p = expf(zr[e] - mx); s[e] = p; sum += p; }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
    } else {
        for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-zr[e]));
    }
    __syncwarp();
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
        float m1 = -CUDART_INF_F, m2 = -CUDART_INF_F;
        for (int e = g * per; e < (g + 1) * per; ++e) {
            const float c = s[e] + (correction ? correction[e] : 0.f);
            if (c > m1) { m2 = m1; m1 = c; } else if (c > m2) m2 = c;
        }
        gs[g] = (group_score == 1 && per > 1) ? m1 + m2 : m1;
        g_open[g] = 0.f;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
        float bv = -CUDART_INF_F;
        int bi = 0x7fffffff;
        for (int g = lane; g < groups; g += 32)
            if (g_open[g] == 0.f && (bi == 0x7fffffff || gs[g] > bv)) { bv = gs[g]; bi = g; }
        warp_argmax(bv, bi);
        if (lane == 0 && bi < groups) g_open[bi] = 1.f;
        __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
        a[e] = g_open[e / per] != 0.f ? s[e] + (correction ? correction[e] : 0.f) : -CUDART_INF_F;
    __syncwarp();
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -CUDART_INF_F;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32)
            if (a[e] > bv) { bv = a[e]; bi = e; }
        warp_argmax(bv, bi);
        if (bi >= E) bi = 0;                   // cannot happen: top <= keep * per open experts with finite scores
        const float w = s[bi];
        total += w;
        if (lane == 0) { ids[(size_t)t * top + k] = bi; wts[(size_t)t * top + k] = w; a[bi] = -CUDART_INF_F; }
        __syncwarp();
    }
    if (renorm) {
        const float inv = 1.0f / (total + 1e-20f);
        __syncwarp();
        for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] *= inv;
    }
}

// One block: rows sorted by expert.  seg[e] .. seg[e+1] are expert e's rows; row_of[entry] is
// the row of (token, choice) = entry; src_tok[row] its token; the row tiles of row_tile rows
// (64 for the plain grouped kernel, 128 for the tensor-core one) are listed as (expert, first row) with their count in n_tiles.
__global__ void moe_plan_kernel(const int* ids, int entries, int top, int E, int row_tile, int* __restrict__ seg,
                                int* __restrict__ row_of, int* __restrict__ src_tok, int* __restrict__ tile_expert,
                                int* __restrict__ tile_row0, int* __restrict__ n_tiles) {
    pdl_prologue();
    ids = pdl_fresh(ids);
    extern __shared__ int shi[];
    int* counts = shi;
    int* offs = shi + E;
    int* cursor = offs + E + 1;
    for (int e = threadIdx.x; e < E; e += blockDim.x) { counts[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int i = threadIdx.x; i < entries; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            offs[e] = run;
            seg[e] = run;
            for (int r0 = 0; r0 < counts[e]; r0 += row_tile) {
                tile_expert[nt] = e;
                tile_row0[nt] = run + r0;
                ++nt;
            }
            run += counts[e];
        }
        offs[E] = run;
        seg[E] = run;
        n_tiles[0] = nt;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < entries; i += blockDim.x) {
        const int e = ids[i];
        const int row = offs[e] + atomicAdd(&cursor[e], 1);
        row_of[i] = row;
        src_tok[row] = i / top;
    }
}

// out rows = A rows x B[e]^T for the row tile's expert e.  B: [E, N, K] row-major.
// GATEUP: two B matrices (gate and up, [E, N, K] each), A rows gathered from x by src_tok, and
// out[row, n] = clamped_glu(gate, up) in type T.  Else: A = rows of `a` in place, out 32-bit.
template <typename T, bool GATEUP>
__global__ void __launch_bounds__(256) moe_grouped_kernel(
    const T* a, const int* src_tok, const T* __restrict__ b0, const T* __restrict__ b1,
    const int* seg, const int* tile_expert, const int* tile_row0,
    const int* n_tiles, void* __restrict__ out, int N, int K, float limit, int act) {
    pdl_prologue();
    a = pdl_fresh(a); src_tok = pdl_fresh(src_tok); seg = pdl_fresh(seg);       // made by the kernels in front
    tile_expert = pdl_fresh(tile_expert); tile_row0 = pdl_fresh(tile_row0); n_tiles = pdl_fresh(n_tiles);
    if ((int)blockIdx.y >= n_tiles[0]) return;
    __shared__ float As[MOE_BK][MOE_BM + 1];
    __shared__ float Bs[GATEUP ? 2 : 1][MOE_BK][MOE_BN + 1];
    __shared__ int s_src[MOE_BM];
    const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y];
    const int rows = min(MOE_BM, seg[e + 1] - row0);
    const int n0 = blockIdx.x * MOE_BN;
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    if (tid < MOE_BM) s_src[tid] = tid < rows ? (GATEUP ? src_tok[row0 + tid] : row0 + tid) : -1;
    __syncthreads();
    const T* B0 = b0 + (size_t)e * N * K;
    const T* B1 = GATEUP ? b1 + (size_t)e * N * K : nullptr;
    float acc0[4][4] = {}, acc1[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
        for (int idx = tid; idx < MOE_BM * MOE_BK; idx += 256) {
            const int r = idx / MOE_BK, kk = idx - r * MOE_BK;
            const int src = s_src[r];
            As[kk][r] = (src >= 0 && k0 + kk < K) ? to_float(a[(size_t)src * K + k0 + kk]) : 0.f;
        }
        for (int idx = tid; idx < MOE_BN * MOE_BK; idx += 256) {
            const int n = idx / MOE_BK, kk = idx - n * MOE_BK;
            const bool ok = n0 + n < N && k0 + kk < K;
            Bs[0][kk][n] = ok ? to_float(B0[(size_t)(n0 + n) * K + k0 + kk]) : 0.f;
            if (GATEUP) Bs[1][kk][n] = ok ? to_float(B1[(size_t)(n0 + n) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_BK; ++kk) {
            float av[4], bv[4], cv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { bv[j] = Bs[0][kk][tx * 4 + j]; if (GATEUP) cv[j] = Bs[1][kk][tx * 4 + j]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc0[i][j] += av[i] * bv[j];
                    if (GATEUP) acc1[i][j] += av[i] * cv[j];
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            if (GATEUP) ((T*)out)[(size_t)(row0 + r) * N + n] = from_float<T>(clamped_glu(acc0[i][j], acc1[i][j], limit, act));
            else ((float*)out)[(size_t)(row0 + r) * N + n] = acc0[i][j];
        }
    }
}

// The same grouped product for bfloat16 on tensor cores: mma.sync m16n8k16 with 32-bit accumulation,
// operands staged through a three-stage cp.async ring in shared memory (rows padded to 40 elements so
// that the 32-bit fragment loads of a warp fall into 32 different banks).  A block takes 128 rows of one
// expert (the plan is made with that row tile) and 128 rows of B: 64 columns of gate and the same 64 of up
// when GATEUP, else 128 output columns.  Eight warps in a 2 x 4 grid, each 64 rows x 32 rows of B (16 gate +
// 16 up columns, so that a thread holds both halves of an output).  Needs K % 8 == 0 (16-byte copies).  Rows
// past the expert's last row and columns past N are filled with zeros by the copies and not stored.
constexpr int MMA_BM = 128, MMA_BR = 128, MMA_BK = 32, MMA_LD = 40, MMA_STAGES = 3;
constexpr size_t MMA_SMEM = (size_t)MMA_STAGES * (MMA_BM + MMA_BR) * MMA_LD * sizeof(bf16);

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool GATEUP>
__global__ void __launch_bounds__(256) moe_grouped_mma_kernel(
    const bf16* a, const int* src_tok, const bf16* __restrict__ b0,
    const bf16* __restrict__ b1, const int* seg, const int* tile_expert,
    const int* tile_row0, const int* n_tiles, void* __restrict__ out, int N, int K,
    float limit, int act) {
    pdl_prologue();
    a = pdl_fresh(a); src_tok = pdl_fresh(src_tok); seg = pdl_fresh(seg);       // made by the kernels in front
    tile_expert = pdl_fresh(tile_expert); tile_row0 = pdl_fresh(tile_row0); n_tiles = pdl_fresh(n_tiles);
    if ((int)blockIdx.y >= n_tiles[0]) return;
    extern __shared__ __align__(16) unsigned char mma_smem[];
    typedef bf16 (*Tile)[MMA_BM][MMA_LD];                      // [stage][row][k]
    Tile As = reinterpret_cast<Tile>(mma_smem);
    Tile Bs = reinterpret_cast<Tile>(mma_smem + (size_t)MMA_STAGES * MMA_BM * MMA_LD * sizeof(bf16));
    static_assert(MMA_BM == MMA_BR, "A and B tiles share a shape");
    constexpr int COLS = GATEUP ? MMA_BR / 2 : MMA_BR;          // output columns of a block
    const int e = tile_expert[blockIdx.y], row0 = tile_row0[blockIdx.y];
    const int rows = min(MMA_BM, seg[e + 1] - row0);
    const int n0 = blockIdx.x * COLS;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3, g = lane >> 2, t4 = lane & 3;
    // this thread's copies: rows tid / 4 and tid / 4 + 64 (of A and of B), 16-byte chunk tid % 4 of a stage's 32 columns.
    // Row r of the B tile: GATEUP: warp wn's 32 rows are gate columns [16 wn, 16 wn + 16) then the same up columns;
    // else output column r.
    const int lr = tid >> 2, lc = (tid & 3) * 8;
    const bf16* a_row[2];
    const bf16* b_row[2];
    bool a_ok[2], b_ok[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int r = lr + 64 * q;
        a_ok[q] = r < rows;
        const int src = a_ok[q] ? (GATEUP ? src_tok[row0 + r] : row0 + r) : 0;
        a_row[q] = a + (size_t)src * K;
        int col;
        const bf16* base = b0;
        if (GATEUP) {
            const int w = r >> 5, in = r & 31;
            col = n0 + w * 16 + (in & 15);
            if (in >= 16) base = b1;
        } else {
            col = n0 + r;
        }
        b_ok[q] = col < N;
        b_row[q] = base + ((size_t)e * N + (b_ok[q] ? col : 0)) * K;
    }
    const int KT = (K + MMA_BK - 1) / MMA_BK;
    auto load = [&](int stage, int kt) {
        const int k = kt * MMA_BK + lc;
        const bool in = k < K;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            cp_async16(&As[stage][lr + 64 * q][lc], a_row[q] + (in ? k : 0), in && a_ok[q]);
            cp_async16(&Bs[stage][lr + 64 * q][lc], b_row[q] + (in ? k : 0), in && b_ok[q]);
        }
    };
    float acc[4][4][4] = {};
    for (int s = 0; s < MMA_STAGES - 1; ++s) {
        if (s < KT) load(s, s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < KT; ++kt) {
        asm volatile("cp.async.wait_group %0;" ::"n"(MMA_STAGES - 2) : "memory");
        __syncthreads();
        const int nxt = kt + MMA_STAGES - 1;
        if (nxt < KT) load(nxt % MMA_STAGES, nxt);
        asm volatile("cp.async.commit_group;" ::: "memory");
        const int st = kt % MMA_STAGES;
#pragma unroll
        for (int kk = 0; kk < MMA_BK; kk += 16) {
            uint32_t bfr[4][2];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int n = wn * 32 + nt * 8 + g;
                bfr[nt][0] = *reinterpret_cast<const uint32_t*>(&Bs[st][n][kk + 2 * t4]);
                bfr[nt][1] = *reinterpret_cast<const uint32_t*>(&Bs[st][n][kk + 8 + 2 * t4]);
            }
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                const int r = wm * 64 + mt * 16 + g;
                uint32_t af[4];
                af[0] = *reinterpret_cast<const uint32_t*>(&As[st][r][kk + 2 * t4]);
                af[1] = *reinterpret_cast<const uint32_t*>(&As[st][r + 8][kk + 2 * t4]);
                af[2] = *reinterpret_cast<const uint32_t*>(&As[st][r][kk + 8 + 2 * t4]);
                af[3] = *reinterpret_cast<const uint32_t*>(&As[st][r + 8][kk + 8 + 2 * t4]);
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) mma_bf16_16816(acc[mt][nt], af, bfr[nt][0], bfr[nt][1]);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int r = wm * 64 + mt * 16 + g + (c >> 1) * 8;
            if (r >= rows) continue;
            if (GATEUP) {
                // B rows 0..15 of the warp are gate (n tiles 0, 1), rows 16..31 the same columns of up (n tiles 2, 3)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int n = n0 + wn * 16 + nt * 8 + 2 * t4 + (c & 1);
                    if (n < N)
                        ((bf16*)out)[(size_t)(row0 + r) * N + n] =
                            __float2bfloat16_rn(clamped_glu(acc[mt][nt][c], acc[mt][nt + 2][c], limit, act));
                }
            } else {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int n = n0 + wn * 32 + nt * 8 + 2 * t4 + (c & 1);
                    if (n < N) ((float*)out)[(size_t)(row0 + r) * N + n] = acc[mt][nt][c];
                }
            }
        }
}

// y[t, f] = clamped_glu(gu[t, f], gu[t, F + f])
template <typename T>
__global__ void clamped_glu_kernel(const T* gu, T* __restrict__ y, int F, float limit, size_t total) {
    pdl_prologue();
    gu = pdl_fresh(gu);
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / F;
    const int f = (int)(idx - t * F);
    y[idx] = from_float<T>(clamped_glu(to_float(gu[t * 2 * F + f]), to_float(gu[t * 2 * F + F + f]), limit));
}

// residual[t,:] += mult * (sum_k wts[t,k] * rows[row_of[t*top+k],:] + shared[t,:])
__global__ void moe_combine_kernel(float* __restrict__ residual, const float* rows,
                                   const int* row_of, const float* wts,
                                   const float* shared, float mult, int top, int W) {
    pdl_prologue();
    rows = pdl_fresh(rows); row_of = pdl_fresh(row_of); wts = pdl_fresh(wts); shared = pdl_fresh(shared);
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k)
            acc += wts[(size_t)t * top + k] * rows[(size_t)row_of[(size_t)t * top + k] * W + i];
        if (shared) acc += shared[(size_t)t * W + i];
        residual[(size_t)t * W + i] += mult * acc;
    }
}

}  // namespace ff

using namespace ff;

// rows of a row tile: of the tensor-core kernel (bfloat16, K % 8 == 0) or of the plain one
FF_EXPORT int ff_moe_row_tile(int tensor_cores) { return tensor_cores ? MMA_BM : MOE_BM; }

FF_EXPORT int ff_moe_route(const float* z, const float* correction, int T, int E, int top, int groups, int keep,
                           int score, int group_score, int renorm, int* ids, float* wts, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
        top > keep * (E / groups))
        return FF_ERR_BAD_ARG;
    const int warps = 4;
    const size_t smem = (size_t)warps * (2 * E + 2 * groups) * sizeof(float);
    if (smem > 48 * 1024) return FF_ERR_UNSUPPORTED;
    FF_LAUNCH(moe_route_kernel, (T + warps - 1) / warps, warps * 32, smem, stream, z, correction, T, E, top, groups, keep, score,
              group_score, renorm, ids, wts);
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_moe_plan(const int* ids, int entries, int top, int E, int row_tile, int* seg, int* row_of,
                          int* src_tok, int* tile_expert, int* tile_row0, int* n_tiles, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (row_tile != MOE_BM && row_tile != MMA_BM) return FF_ERR_BAD_ARG;
    const size_t smem = (size_t)(3 * E + 1) * sizeof(int);
    if (smem > 48 * 1024) return FF_ERR_UNSUPPORTED;
    FF_LAUNCH(moe_plan_kernel, 1, 1024, smem, stream, ids, entries, top, E, row_tile, seg, row_of, src_tok, tile_expert,
              tile_row0, n_tiles);
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_moe_grouped(const void* a, const int* src_tok, const void* b0, const void* b1, int dtype, int gateup,
                             const int* seg, const int* tile_expert, const int* tile_row0, const int* n_tiles,
                             void* out, int max_tiles, int N, int K, float limit, int act, int tensor_cores,
                             cudaStream_t stream) {
    if (max_tiles <= 0) return 0;
    if (tensor_cores) {
        // the plan was made with 128-row tiles
        if (dtype != 1 || K % 8 || ((((uintptr_t)a | (uintptr_t)b0 | (uintptr_t)b1) & 15) != 0)) return FF_ERR_BAD_ARG;
        const int cols = gateup ? MMA_BR / 2 : MMA_BR;
        dim3 grid((N + cols - 1) / cols, max_tiles);
        if (gateup) {
            FF_SMEM_LIMIT((moe_grouped_mma_kernel<true>), MMA_SMEM);
            FF_LAUNCH((moe_grouped_mma_kernel<true>), grid, 256, MMA_SMEM, stream, (const bf16*)a, src_tok, (const bf16*)b0,
                      (const bf16*)b1, seg, tile_expert, tile_row0, n_tiles, out, N, K, limit, act);
        } else {
            FF_SMEM_LIMIT((moe_grouped_mma_kernel<false>), MMA_SMEM);
            FF_LAUNCH((moe_grouped_mma_kernel<false>), grid, 256, MMA_SMEM, stream, (const bf16*)a, src_tok, (const bf16*)b0,
                      (const bf16*)b1, seg, tile_expert, tile_row0, n_tiles, out, N, K, limit, act);
        }
        FF_LAUNCH_CHECK();
        return 0;
    }
    dim3 grid((N + MOE_BN - 1) / MOE_BN, max_tiles);
#define FF_MOE(T, G)                                                                                               \
    FF_LAUNCH((moe_grouped_kernel<T, G>), grid, 256, 0, stream, (const T*)a, src_tok, (const T*)b0, (const T*)b1, seg, \
              tile_expert, tile_row0, n_tiles, out, N, K, limit, act)
    if (dtype == 0 && gateup) FF_MOE(float, true);
    else if (dtype == 0) FF_MOE(float, false);
    else if (dtype == 1 && gateup) FF_MOE(bf16, true);
    else if (dtype == 1) FF_MOE(bf16, false);
    else return FF_ERR_BAD_ARG;
#undef FF_MOE
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_clamped_glu(const void* gu, void* y, int dtype, int T, int F, float limit, cudaStream_t stream) {
    const size_t total = (size_t)T * F;
    if (total == 0) return 0;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) FF_LAUNCH((clamped_glu_kernel<float>), blocks, 256, 0, stream, (const float*)gu, (float*)y, F, limit, total);
    else if (dtype == 1) FF_LAUNCH((clamped_glu_kernel<bf16>), blocks, 256, 0, stream, (const bf16*)gu, (bf16*)y, F, limit, total);
    else return FF_ERR_BAD_ARG;
    FF_LAUNCH_CHECK();
    return 0;
}

FF_EXPORT int ff_moe_combine(float* residual, const float* rows, const int* row_of, const float* wts,
                             const float* shared, float mult, int T, int top, int W, cudaStream_t stream) {
    if (T <= 0) return 0;
    FF_LAUNCH(moe_combine_kernel, T, W >= 1024 ? 256 : 128, 0, stream, residual, rows, row_of, wts, shared, mult, top, W);
    FF_LAUNCH_CHECK();
    return 0;
}
