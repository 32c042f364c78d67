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

__device__ __forceinline__ void store_row4(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void store_row4(bf16* p, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = pk;
}

// S: the number of streams at compile time (1 to 8: every loop over the streams unrolls and the
// weights sit in registers), or 0 for any number up to kMaxStreams.  V: elements per thread and
// access (4: the row's width is a multiple of 4 and every pointer 16-byte aligned; else 1).
template <typename T, int S_, int V>
__global__ void __launch_bounds__(kThreads)
streams_step_kernel(float* __restrict__ streams, int64_t stream_stride, const float* __restrict__ init,
                    const float* __restrict__ y, const float* __restrict__ mix, const float* __restrict__ outw,
                    const float* __restrict__ inw, const float* __restrict__ gain, float eps, T* __restrict__ normed,
                    float* __restrict__ total, int d, int s_runtime) {
    constexpr int SM = S_ > 0 ? S_ : kMaxStreams;
    const int S = S_ > 0 ? S_ : s_runtime;
    extern __shared__ __align__(16) float us[];              // [d]: the row that is read, until its norm is known
    __shared__ float red[32];
    // the streams' weights are model tensors: no kernel of the step writes them
    float w_mix[SM][SM], w_out[SM], w_in[SM];
#pragma unroll
    for (int a = 0; a < SM; a++) {
        w_out[a] = (y && a < S) ? outw[a] : 0.f;
        w_in[a] = (inw && a < S) ? inw[a] : 0.f;
#pragma unroll
        for (int b = 0; b < SM; b++) w_mix[a][b] = (y && a < S && b < S) ? mix[a * S + b] : 0.f;
    }
    griddep_wait();
    griddep_launch();
    const int64_t row = (int64_t)blockIdx.x * d;
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < d; c += kThreads * V) {
        float old[SM][V], cur[SM][V], yv[V];
        if (init) {
            float tmp[V];
            if constexpr (V == 4) *reinterpret_cast<float4*>(tmp) = *reinterpret_cast<const float4*>(init + row + c);
            else tmp[0] = init[row + c];
#pragma unroll
            for (int s = 0; s < SM; s++)
#pragma unroll
                for (int v = 0; v < V; v++) old[s][v] = tmp[v];
        } else {
#pragma unroll
            for (int s = 0; s < SM; s++)
                if (s < S) {
                    if constexpr (V == 4)
                        *reinterpret_cast<float4*>(old[s]) = *reinterpret_cast<const float4*>(streams + s * stream_stride + row + c);
                    else old[s][0] = streams[s * stream_stride + row + c];
                }
        }
        if (y) {
            if constexpr (V == 4) *reinterpret_cast<float4*>(yv) = *reinterpret_cast<const float4*>(y + row + c);
            else yv[0] = y[row + c];
#pragma unroll
            for (int t = 0; t < SM; t++)
                if (t < S) {
#pragma unroll
                    for (int v = 0; v < V; v++) {
                        float acc = 0.f;
#pragma unroll
                        for (int s = 0; s < SM; s++)
                            if (s < S) acc += w_mix[s][t] * old[s][v];
                        cur[t][v] = acc + w_out[t] * yv[v];
                    }
                }
        } else {
#pragma unroll
            for (int t = 0; t < SM; t++)
#pragma unroll
                for (int v = 0; v < V; v++) cur[t][v] = old[t][v];
        }
        if (y || init) {
#pragma unroll
            for (int t = 0; t < SM; t++)
                if (t < S) {
                    if constexpr (V == 4)
                        *reinterpret_cast<float4*>(streams + t * stream_stride + row + c) = *reinterpret_cast<float4*>(cur[t]);
                    else streams[t * stream_stride + row + c] = cur[t][0];
                }
        }
        if (inw) {
#pragma unroll
            for (int v = 0; v < V; v++) {
                float u = 0.f;
#pragma unroll
                for (int t = 0; t < SM; t++)
                    if (t < S) u += w_in[t] * cur[t][v];
                us[c + v] = u;
                ss += u * u;
            }
        }
        if (total) {
            float tv[V];
#pragma unroll
            for (int v = 0; v < V; v++) {
                float a = 0.f;
#pragma unroll
                for (int t = 0; t < SM; t++)
                    if (t < S) a += cur[t][v];
                tv[v] = a;
            }
            if constexpr (V == 4) *reinterpret_cast<float4*>(total + row + c) = *reinterpret_cast<float4*>(tv);
            else total[row + c] = tv[0];
        }
    }
    if (!inw) return;
    ss = block_sum(ss, red);
    const float scale = rsqrtf(ss / (float)d + eps);
    // a thread scales the elements it wrote itself: no barrier between the two loops is needed
    for (int c = threadIdx.x * V; c < d; c += kThreads * V) {
        if constexpr (V == 4) {
            const float4 u = *reinterpret_cast<const float4*>(us + c), g = *reinterpret_cast<const float4*>(gain + c);
            store_row4(normed + row + c, u.x * scale * g.x, u.y * scale * g.y, u.z * scale * g.z, u.w * scale * g.w);
        } else {
            normed[row + c] = from_f32<T>(us[c] * scale * gain[c]);
        }
    }
}

template <typename T, int S_, int V>
int launch_streams(float* streams, int64_t stream_stride, const float* init, const float* y, const float* mix,
                   const float* outw, const float* inw, const float* gain, float eps, void* normed, float* total, int n,
                   int d, int S, size_t smem, cudaStream_t s) {
    auto kern = streams_step_kernel<T, S_, V>;
    static size_t raised = 48 * 1024;
    if (smem > raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) KLLM_FAIL("residual streams: shared memory limit: %s", cudaGetErrorString(e));
        raised = smem;
    }
    kllm_launch(kern, dim3(n), dim3(kThreads), smem, s, streams, stream_stride, init, y, mix, outw, inw, gain, eps,
                (T*)normed, total, d, S);
    KLLM_LAUNCH_STATUS();
}

template <typename T, int V>
int pick_streams(float* streams, int64_t stream_stride, const float* init, const float* y, const float* mix,
                 const float* outw, const float* inw, const float* gain, float eps, void* normed, float* total, int n,
                 int d, int S, size_t smem, cudaStream_t s) {
#define KLLM_STREAMS_S(N)                                                                                              \
    if (S == N)                                                                                                        \
        return launch_streams<T, N, V>(streams, stream_stride, init, y, mix, outw, inw, gain, eps, normed, total, n, d, S, \
                                       smem, s)
    KLLM_STREAMS_S(1); KLLM_STREAMS_S(2); KLLM_STREAMS_S(3); KLLM_STREAMS_S(4);
    KLLM_STREAMS_S(5); KLLM_STREAMS_S(6); KLLM_STREAMS_S(7); KLLM_STREAMS_S(8);
#undef KLLM_STREAMS_S
    return launch_streams<T, 0, 1>(streams, stream_stride, init, y, mix, outw, inw, gain, eps, normed, total, n, d, S, smem, s);
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
    // 16-byte accesses where every row of every operand allows them
    const uintptr_t addr = (uintptr_t)streams | (uintptr_t)init | (uintptr_t)y | (uintptr_t)total | (uintptr_t)normed |
                           (uintptr_t)gain;
    const bool vec = d % 4 == 0 && stream_stride % 4 == 0 && addr % 16 == 0;
    if (dtype != KLLM_F32 && dtype != KLLM_BF16) KLLM_FAIL("residual streams: unknown element type %d", dtype);
#define KLLM_STREAMS(T, V) \
    return pick_streams<T, V>(streams, stream_stride, init, y, mix, outw, inw, gain, eps, normed, total, n, d, S, smem, s)
    if (dtype == KLLM_F32) {
        if (vec) KLLM_STREAMS(float, 4);
        KLLM_STREAMS(float, 1);
    }
    if (vec) KLLM_STREAMS(bf16, 4);
    KLLM_STREAMS(bf16, 1);
#undef KLLM_STREAMS
}
