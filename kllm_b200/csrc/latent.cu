// Between the down-projections and the attention of a layer that attends through low-rank
// latents: one kernel per step that takes the float32 result of the stacked product
// [query latent (Rq values) | key/value latent (R values)] of every token and
//
//   cq[t,:] = a[t,:]  * rsqrt(mean(a[t,:]^2) + eps) * q_gain        stored dense, model dtype
//   c[t,:]  = b[t,:]  * rsqrt(mean(b[t,:]^2) + eps) * kv_gain       stored in the paged cache
//
// The key/value latent is the only thing such a layer caches: a store of one "head" of R
// values per token, [pages][1][page_size][R], written at position p_t of the token's request.
// Sums of squares and scales are float32.  A layer that reads another layer's latents has
// no second segment (cache NULL).  One CTA per token; the order of a row's additions
// depends on its width alone.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(latent)

namespace {

constexpr int kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads)
latent_norm_append_kernel(T* __restrict__ q_out, const float* __restrict__ proj, int64_t proj_stride,
                          const float* __restrict__ q_gain, const float* __restrict__ kv_gain, float eps,
                          const int* __restrict__ positions, const int* __restrict__ token_req,
                          const int* __restrict__ block_table, int max_blocks, T* __restrict__ cache, int Rq, int R,
                          int page_size) {
    __shared__ float red[32];
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x;
    const float* a = proj + (int64_t)t * proj_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < Rq; i += kThreads) ss += a[i] * a[i];
    ss = block_sum(ss, red);
    float scale = rsqrtf(ss / (float)Rq + eps);
    T* qo = q_out + (int64_t)t * Rq;
    for (int i = threadIdx.x; i < Rq; i += kThreads) qo[i] = from_f32<T>(a[i] * scale * q_gain[i]);

    if (cache == nullptr) return;
    const float* b = a + Rq;
    ss = 0.f;
    for (int i = threadIdx.x; i < R; i += kThreads) ss += b[i] * b[i];
    ss = block_sum(ss, red);
    scale = rsqrtf(ss / (float)R + eps);
    const int p = positions[t];
    const int lp = p / page_size, slot = p - lp * page_size;
    const int64_t page = block_table[(int64_t)token_req[t] * max_blocks + lp];
    if (page < 0) return;                                   // a table without a page here: checked on the host
    T* row = cache + (page * page_size + slot) * R;
    for (int i = threadIdx.x; i < R; i += kThreads) row[i] = from_f32<T>(b[i] * scale * kv_gain[i]);
}

}  // namespace

// proj float32 [n][Rq (+ R)] at row stride proj_stride; q_out [n][Rq] contiguous in the element
// type `dtype`, which is also the cache's.  cache NULL: proj holds the query latents alone.
extern "C" int kllm_latent_norm_append(void* q_out, const float* proj, int64_t proj_stride, const float* q_gain,
                                       const float* kv_gain, float eps, const int* positions, const int* token_req,
                                       const int* block_table, int max_blocks, void* cache, int n, int Rq, int R,
                                       int page_size, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (Rq <= 0 || (cache && R <= 0)) KLLM_FAIL("latent norm: latent sizes %d and %d", Rq, R);
    if (cache && (page_size <= 0 || !block_table || !kv_gain)) KLLM_FAIL("latent norm: cache without pages, table or gain");
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KLLM_F32)
        kllm_launch((latent_norm_append_kernel<float>), dim3(n), dim3(kThreads), 0, s, (float*)q_out, proj, proj_stride,
                    q_gain, kv_gain, eps, positions, token_req, block_table, max_blocks, (float*)cache, Rq, R, page_size);
    else if (dtype == KLLM_BF16)
        kllm_launch((latent_norm_append_kernel<bf16>), dim3(n), dim3(kThreads), 0, s, (bf16*)q_out, proj, proj_stride,
                    q_gain, kv_gain, eps, positions, token_req, block_table, max_blocks, (bf16*)cache, Rq, R, page_size);
    else
        KLLM_FAIL("latent norm: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}
