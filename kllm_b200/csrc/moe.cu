// Routed experts: every token runs `top` of E small gated feed-forwards.
//
//   route     z = W_r h in float32 (h widened from the model's element type), score =
//             sigmoid(z) or softmax(z); the `top` largest scores, the lower index first among
//             equals; the weights are the chosen scores, as they are or divided by their sum.
//   sort      the (token, choice) pairs ordered by expert: offsets[E + 1] and perm[n * top]
//             (sorted row -> token * top + choice), on the device, so that a step's launch
//             shapes do not depend on the routing.
//   gemm      for the sorted rows of every expert e, C = A W_e^T as tiles of 32 rows x 64
//             columns with float32 accumulation on the CUDA cores.  Two forms:
//             "gated" reads row `token` of the layer's input, times the row's weight if the
//             weight acts on the expert's input, and stores act(gate) * up per sorted row;
//             "down" reads the sorted rows and stores row token * top + choice of a float32
//             matrix, times the weight if it acts on the output.
//   combine   y[t] = sum over the choices of a token, in choice order.
//
// A row's sums do not depend on which other rows share its tile or its launch.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(moe)

namespace {

// ---- router ----------------------------------------------------------------------
// one warp per token; E logits in shared memory (E <= 1024).
template <typename T>
__global__ void __launch_bounds__(128)
route_kernel(int* __restrict__ idx, float* __restrict__ wt, const T* __restrict__ h, const float* __restrict__ router,
             int n, int d, int E, int top, int softmax, int renorm) {
    extern __shared__ float zsh[];            // [4 warps][E]
    griddep_wait();
    griddep_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + warp;
    if (t >= n) return;
    float* z = zsh + warp * E;
    const T* hr = h + (int64_t)t * d;
    for (int e = 0; e < E; e++) {
        const float* wr = router + (int64_t)e * d;
        float acc = 0.f;
        for (int c = lane; c < d; c += 32) acc += to_f32(hr[c]) * wr[c];
        acc = warp_sum(acc);
        if (lane == 0) z[e] = acc;
    }
    __syncwarp();
    if (softmax) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) sum += expf(z[e] - m);
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) z[e] = expf(z[e] - m) / sum;
    } else {
        for (int e = lane; e < E; e += 32) z[e] = 1.f / (1.f + expf(-z[e]));
    }
    __syncwarp();
    float total = 0.f;
    for (int c = 0; c < top; c++) {
        float best = -INFINITY;
        int bi = E;
        for (int e = lane; e < E; e += 32)
            if (z[e] > best) { best = z[e]; bi = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == 0) {
            idx[(int64_t)t * top + c] = bi;
            wt[(int64_t)t * top + c] = best;
            z[bi] = -INFINITY;
        }
        total += best;
        __syncwarp();
    }
    if (renorm && lane == 0)
        for (int c = 0; c < top; c++) wt[(int64_t)t * top + c] /= total;
}

// ---- sort by expert ---------------------------------------------------------------
// one CTA; counts and offsets in shared memory.  The order of the rows inside an expert is
// whatever the atomics give: no result depends on it.
__global__ void __launch_bounds__(1024)
sort_kernel(int* __restrict__ offsets, int* __restrict__ perm, int* __restrict__ rank, const int* __restrict__ idx,
            int rows, int E) {
    extern __shared__ int cnt[];              // [E + 1]
    griddep_wait();
    griddep_launch();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int r = threadIdx.x; r < rows; r += blockDim.x) rank[r] = atomicAdd(&cnt[idx[r]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; e++) {
            const int c = cnt[e];
            cnt[e] = run;
            run += c;
        }
        cnt[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = cnt[e];
    for (int r = threadIdx.x; r < rows; r += blockDim.x) perm[cnt[idx[r]] + rank[r]] = r;
}

// ---- the experts' products ---------------------------------------------------------
constexpr int BM = 32, BN = 64, BK = 32, GT = 256;

__device__ __forceinline__ float act_silu(float g) { return g / (1.f + expf(-g)); }

// GATED: W_e is [2 * N][K] (gate rows, then up rows), C [rows][N] in T, sorted order.
// else : W_e is [N][K], C float32 [rows][N] at row perm[r].
template <typename T, bool GATED>
__global__ void __launch_bounds__(GT)
expert_gemm_kernel(void* __restrict__ c_out, const T* __restrict__ a, int64_t a_stride, const T* __restrict__ w,
                   const int* __restrict__ offsets, const int* __restrict__ perm, const float* __restrict__ wt,
                   int E, int top, int N, int K, int scale_in, int scale_out) {
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[GATED ? 2 : 1][BK][BN + 1];
    __shared__ int srow[BM];
    __shared__ float sscale[BM];
    griddep_wait();
    griddep_launch();
    // which expert and which of its row tiles
    int tile = blockIdx.y, e = 0, lo = 0, hi = 0;
    for (; e < E; e++) {
        lo = offsets[e];
        hi = offsets[e + 1];
        const int nt = (hi - lo + BM - 1) / BM;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e >= E) return;
    const int r0 = lo + tile * BM, nr = min(BM, hi - r0);
    const int n0 = blockIdx.x * BN;
    const int tid = threadIdx.x;
    if (tid < BM) {
        int src = 0;
        float sc = 1.f;
        if (tid < nr) {
            const int flat = perm[r0 + tid];
            src = GATED ? flat / top : r0 + tid;
            if (GATED ? scale_in : scale_out) sc = wt[flat];
        }
        srow[tid] = src;
        sscale[tid] = sc;
    }
    __syncthreads();
    const T* we = w + (int64_t)e * (GATED ? 2 : 1) * N * K;
    const int ty = tid / 16, tx = tid % 16;                 // rows ty, ty + 16; columns tx + 16 j
    float acc[GATED ? 2 : 1][2][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = tid; i < BM * BK; i += GT) {
            const int rr = i / BK, kk = i - rr * BK;
            float v = 0.f;
            if (rr < nr && k0 + kk < K) {
                v = to_f32(a[(int64_t)srow[rr] * a_stride + k0 + kk]);
                if (GATED) v *= sscale[rr];
            }
            As[kk][rr] = v;
        }
        for (int i = tid; i < BN * BK; i += GT) {
            const int cc = i / BK, kk = i - cc * BK;
            const bool ok = n0 + cc < N && k0 + kk < K;
            Ws[0][kk][cc] = ok ? to_f32(we[(int64_t)(n0 + cc) * K + k0 + kk]) : 0.f;
            if (GATED) Ws[1][kk][cc] = ok ? to_f32(we[(int64_t)(N + n0 + cc) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < BK; kk++) {
            const float a0 = As[kk][ty], a1 = As[kk][ty + 16];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float b = Ws[0][kk][tx + 16 * j];
                acc[0][0][j] += a0 * b;
                acc[0][1][j] += a1 * b;
                if (GATED) {
                    const float b2 = Ws[1][kk][tx + 16 * j];
                    acc[1][0][j] += a0 * b2;
                    acc[1][1][j] += a1 * b2;
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int rr = ty + 16 * i;
        if (rr >= nr) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int cc = n0 + tx + 16 * j;
            if (cc >= N) continue;
            if (GATED) {
                ((T*)c_out)[(int64_t)(r0 + rr) * N + cc] = from_f32<T>(act_silu(acc[0][i][j]) * acc[GATED ? 1 : 0][i][j]);
            } else {
                ((float*)c_out)[(int64_t)perm[r0 + rr] * N + cc] = acc[0][i][j] * sscale[rr];
            }
        }
    }
}

__global__ void __launch_bounds__(256)
combine_kernel(float* __restrict__ y, const float* __restrict__ parts, int64_t total, int d, int top) {
    griddep_wait();
    griddep_launch();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / d;
        const int c = (int)(i - t * d);
        float s = 0.f;
        for (int j = 0; j < top; j++) s += parts[(t * top + j) * d + c];
        y[i] = s;
    }
}

}  // namespace

// idx int32 [n][top], wt float32 [n][top]; h [n][d] contiguous in `dtype`; router float32 [E][d].
extern "C" int kllm_moe_route(int* idx, float* wt, const void* h, const float* router, int n, int d, int E, int top,
                              int softmax, int renorm, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (E <= 0 || E > 1024 || top <= 0 || top > E) KLLM_FAIL("moe route: %d of %d experts (at most 1024)", top, E);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)4 * E * sizeof(float);
    if (dtype == KLLM_F32)
        kllm_launch((route_kernel<float>), dim3((n + 3) / 4), dim3(128), smem, s, idx, wt, (const float*)h, router, n, d, E,
                    top, softmax, renorm);
    else if (dtype == KLLM_BF16)
        kllm_launch((route_kernel<bf16>), dim3((n + 3) / 4), dim3(128), smem, s, idx, wt, (const bf16*)h, router, n, d, E,
                    top, softmax, renorm);
    else
        KLLM_FAIL("moe route: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}

// offsets int32 [E + 1], perm and rank int32 [rows], idx int32 [rows] with values in [0, E).
extern "C" int kllm_moe_sort(int* offsets, int* perm, int* rank, const int* idx, int rows, int E, void* stream) {
    if (rows <= 0) return 0;
    if (E <= 0 || E > 1024) KLLM_FAIL("moe sort: %d experts (at most 1024)", E);
    kllm_launch((sort_kernel), dim3(1), dim3(1024), (size_t)(E + 1) * sizeof(int), (cudaStream_t)stream, offsets, perm, rank,
                idx, rows, E);
    KLLM_LAUNCH_STATUS();
}

// gated != 0: a [tokens][K] (row stride a_stride), w [E][2N][K], c [rows][N] in `dtype`;
// gated == 0: a [rows][K] sorted, w [E][N][K], c float32 [rows][N] indexed by perm.
extern "C" int kllm_moe_gemm(void* c, const void* a, int64_t a_stride, const void* w, const int* offsets,
                             const int* perm, const float* wt, int rows, int E, int top, int N, int K, int gated,
                             int scale_in, int scale_out, int dtype, void* stream) {
    if (rows <= 0) return 0;
    if (N <= 0 || K <= 0 || E <= 0 || top <= 0) KLLM_FAIL("moe gemm: bad sizes");
    const int row_tiles = (rows + BM - 1) / BM + E;
    if (row_tiles > 65535) KLLM_FAIL("moe gemm: %d rows in one launch", rows);
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((N + BN - 1) / BN, row_tiles);
#define KLLM_MOE(T, G)                                                                                            \
    kllm_launch((expert_gemm_kernel<T, G>), grid, dim3(GT), 0, s, c, (const T*)a, a_stride, (const T*)w, offsets, perm, \
                wt, E, top, N, K, scale_in, scale_out)
    if (dtype == KLLM_F32) {
        if (gated) KLLM_MOE(float, true); else KLLM_MOE(float, false);
    } else if (dtype == KLLM_BF16) {
        if (gated) KLLM_MOE(bf16, true); else KLLM_MOE(bf16, false);
    } else {
        KLLM_FAIL("moe gemm: unknown element type %d", dtype);
    }
#undef KLLM_MOE
    KLLM_LAUNCH_STATUS();
}

extern "C" int kllm_moe_combine(float* y, const float* parts, int n, int d, int top, void* stream) {
    if (n <= 0) return 0;
    const int64_t total = (int64_t)n * d;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    kllm_launch((combine_kernel), dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, y, parts, total, d, top);
    KLLM_LAUNCH_STATUS();
}
