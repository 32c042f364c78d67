// Several residual streams in place of one: a model keeps S copies x_1 .. x_S of the residual
// stream, a sublayer reads a weighted sum of them and its output goes back into every one:
//
//   write   x_t <- sum_s mix[s][t] x_s + out[t] y        all t at once, from the old streams
//   read    u = sum_t in[t] x_t;   normed = u * rsqrt(mean(u^2) + eps) * gain
//   total   x = sum_t x_t                                  the model's output stream
//
// One kernel does any of the three in that order for a row, so that the write of one
// sublayer, the read of the next and its RMS norm are a single pass over the S rows: the
// streams are read once and written once per sublayer.  With `init` the old streams are S
// copies of one row (the embedding's output) and are not read.  Everything is float32; the
// normed row is stored in the model's element type.  One CTA per token row; every sum runs
// over the streams in index order and over the row in an order fixed by its width.
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(streams)

namespace {

constexpr int kThreads = 256;
constexpr int kMaxStreams = 16;

template <typename T>
__global__ void __launch_bounds__(kThreads)
streams_step_kernel(float* __restrict__ streams, int64_t stream_stride, const float* __restrict__ init,
                    const float* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ outw,
                    const float* __restrict__ inw, const float* __restrict__ gain, float eps, T* __restrict__ normed,
                    float* __restrict__ total, int d, int S) {
    extern __shared__ float us[];                            // [d]: the row that is read, until its norm is known
    __shared__ float red[32];
    __shared__ float w_mix[kMaxStreams * kMaxStreams], w_out[kMaxStreams], w_in[kMaxStreams];
    // the streams' weights are model tensors: no kernel of the step writes them
    for (int i = threadIdx.x; i < S * S; i += kThreads) w_mix[i] = y ? mix[i] : 0.f;
    for (int i = threadIdx.x; i < S; i += kThreads) {
        w_out[i] = y ? outw[i] : 0.f;
        w_in[i] = inw ? inw[i] : 0.f;
    }
    griddep_wait();
    griddep_launch();
    __syncthreads();
    const int64_t row = (int64_t)blockIdx.x * d;
    float ss = 0.f;
    for (int c = threadIdx.x; c < d; c += kThreads) {
        float old[kMaxStreams], cur[kMaxStreams];
#pragma unroll
        for (int s = 0; s < kMaxStreams; s++)
            if (s < S) old[s] = init ? init[row + c] : streams[s * stream_stride + row + c];
        if (y) {
            const float yv = y[row + c];
#pragma unroll
            for (int t = 0; t < kMaxStreams; t++)
                if (t < S) {
                    float v = 0.f;
#pragma unroll
                    for (int s = 0; s < kMaxStreams; s++)
                        if (s < S) v += w_mix[s * S + t] * old[s];
                    cur[t] = v + w_out[t] * yv;
                }
        } else {
#pragma unroll
            for (int t = 0; t < kMaxStreams; t++)
                if (t < S) cur[t] = old[t];
        }
        if (y || init) {
#pragma unroll
            for (int t = 0; t < kMaxStreams; t++)
                if (t < S) streams[t * stream_stride + row + c] = cur[t];
        }
        if (inw) {
            float u = 0.f;
#pragma unroll
            for (int t = 0; t < kMaxStreams; t++)
                if (t < S) u += w_in[t] * cur[t];
            us[c] = u;
            ss += u * u;
        }
        if (total) {
            float v = 0.f;
#pragma unroll
            for (int t = 0; t < kMaxStreams; t++)
                if (t < S) v += cur[t];
            total[row + c] = v;
        }
    }
    if (!inw) return;
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)d + eps);
    for (int c = threadIdx.x; c < d; c += kThreads) normed[row + c] = from_f32<T>(us[c] * scale * gain[c]);
}

}  // namespace

// streams float32 [S][n][d] (stream s at s * stream_stride), updated in place.
// init   float32 [n][d] or NULL: the old streams are S copies of it (and are written out);
// y      float32 [n][d] or NULL: a sublayer's output, written into the streams with mix [S][S]
//        (indexed [from][to]) and outw [S];
// inw    float32 [S] or NULL: read the (new) streams with these weights and store the RMS
//        norm of that row, times gain [d], in normed [n][d] of element type `dtype`;
// total  float32 [n][d] or NULL: receives the sum of the (new) streams.
extern "C" int kllm_streams_step(float* streams, int64_t stream_stride, const float* init, const float* y,
                                 const float* mix, const float* outw, const float* inw, const float* gain, float eps,
                                 void* normed, float* total, int n, int d, int S, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (S < 1 || S > kMaxStreams) KLLM_FAIL("residual streams: %d streams (1 to %d)", S, kMaxStreams);
    if (d <= 0 || (size_t)d * sizeof(float) > 200 * 1024) KLLM_FAIL("residual streams: width %d", d);
    if (y && (!mix || !outw)) KLLM_FAIL("residual streams: a write needs its mix and out weights");
    if (inw && (!gain || !normed)) KLLM_FAIL("residual streams: a read needs the norm's gain and a place for the row");
    if (!streams) KLLM_FAIL("residual streams: no streams");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = inw ? (size_t)d * sizeof(float) : 0;
#define KLLM_STREAMS(T)                                                                                           \
    do {                                                                                                          \
        auto kern = streams_step_kernel<T>;                                                                       \
        static size_t raised = 48 * 1024;                                                                         \
        if (smem > raised) {                                                                                      \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
            if (e != cudaSuccess) KLLM_FAIL("residual streams: shared memory limit: %s", cudaGetErrorString(e)); \
            raised = smem;                                                                                        \
        }                                                                                                         \
        kllm_launch(kern, dim3(n), dim3(kThreads), smem, s, streams, stream_stride, init, y, mix, outw, inw, gain, eps, \
                    (T*)normed, total, d, S);                                                                     \
    } while (0)
    if (dtype == KLLM_F32) KLLM_STREAMS(float);
    else if (dtype == KLLM_BF16) KLLM_STREAMS(bf16);
    else KLLM_FAIL("residual streams: unknown element type %d", dtype);
#undef KLLM_STREAMS
    KLLM_LAUNCH_STATUS();
}
