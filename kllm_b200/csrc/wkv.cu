// A linear-attention recurrence with a per-channel decay and a bonus for the current
// token (the time mixing of RWKV-style models), for mixed batches of prompt portions
// and single tokens, with the state of every request in a slot of a state tensor.
//
// Per head, with N key channels i and N value channels j and a state S [N][N] that starts
// at zero for a new request:
//
//     a_ij   = k_i v_j
//     o_j    = sum_i r_i (S_ij + u_i a_ij)          the bonus u acts on the current token only
//     S_ij  <- w_i S_ij + a_ij                       w_i = exp(-exp(z_i + w0_i)) in (0, 1)
//
// Everything here is float32: the inputs r, k, v, z come out of their projections
// unrounded, the decay, the state, the sums.  A token's sums run over i = 0 .. N-1 in
// that order whatever the batch holds and however the prompt was cut, and the state is
// carried through the slot, so a position's result does not depend on the cutting.
//
// Four kernels:
//   shift_mix   m_s = h + (h_prev - h) * mu_s for s = 0 .. n_mix-1, h_prev being the row
//               before in the same request, or the request's last row of the step before
//               (kept in its state slot, zeros at the start); the slot is updated.
//   scan        the recurrence above over the rows of every request.  Heads of 16, 32, 64 or
//               128 channels: a CTA per (head, slice of value channels, request); a thread
//               keeps S[4g .. 4g+3][j] of up to four value channels j in registers, the N/4
//               threads of a value channel are neighbouring lanes and add their parts of o_j
//               by shuffles in a fixed tree; r, k, the decay and u*k of eight rows at a time
//               are staged in shared memory (two buffers, one barrier per eight rows).  Other head sizes
//               up to 128: one CTA per (head, request), thread j owning all of S[.][j].
//               In the slot the state lies as [heads][j][i], so a thread's part is
//               contiguous and a warp's loads are whole lines.
//   decay_outer z = W2 tanh(low): the outer half of the decay's low-rank product, tanh included.
//   gate_norm   y = o / rms(o over the head's N values) * gain * silu(g).
#include "common.cuh"

KLLM_EXPORT_LAST_ERROR(wkv)

namespace {

// ---- token shift ---------------------------------------------------------------
// grid: one CTA per token.  The thread of channel c of a request's FIRST row reads the
// slot's channel c and afterwards writes the request's LAST row there; no other thread
// touches that element, so a one-row request (decode) and a portion behave alike.
template <typename T>
__global__ void __launch_bounds__(256)
shift_mix_kernel(T* __restrict__ out, const T* __restrict__ h, const float* __restrict__ mu, float* __restrict__ state,
                 int64_t state_stride, int64_t prev_off, const int* __restrict__ q_start,
                 const int* __restrict__ token_req, const int* __restrict__ state_slots, int n, int d, int n_mix) {
    griddep_wait();
    griddep_launch();
    const int t = blockIdx.x;
    const int s = token_req[t];
    const int first_row = q_start[s];
    const bool first = t == first_row;
    float* slot = state + (int64_t)state_slots[s] * state_stride + prev_off;
    const T* hr = h + (int64_t)t * d;
    const T* pr = h + (int64_t)(t - 1) * d;
    const T* last = h + (int64_t)(q_start[s + 1] - 1) * d;
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        const float x = to_f32(hr[c]);
        float p;
        if (first) {
            p = slot[c];
            slot[c] = to_f32(last[c]);
        } else {
            p = to_f32(pr[c]);
        }
        const float diff = p - x;
        for (int m = 0; m < n_mix; m++)
            out[((int64_t)m * n + t) * d + c] = from_f32<T>(x + diff * mu[(int64_t)m * d + c]);
    }
}

// ---- the recurrence --------------------------------------------------------------
// blockDim = N rounded up to a warp; thread j < N owns S[0..N-1][j].  The r, k, w, u*k of a
// token are shared through shared memory (two buffers: the next token's values are
// loaded and its decay computed while this token's sums run).
template <int NMAX>
__global__ void __launch_bounds__(NMAX)
wkv_scan_kernel(float* __restrict__ o, int64_t o_stride, const float* __restrict__ r, int64_t r_stride,
                const float* __restrict__ k, int64_t k_stride, const float* __restrict__ v, int64_t v_stride,
                const float* __restrict__ z, int64_t z_stride, const float* __restrict__ w0,
                const float* __restrict__ u, float* __restrict__ state, int64_t state_stride,
                const int* __restrict__ q_start, const int* __restrict__ state_slots, int N) {
    __shared__ float sh[2][4][NMAX];          // r, k, w, u * k
    griddep_wait();
    griddep_launch();
    const int head = blockIdx.x, s = blockIdx.y, j = threadIdx.x;
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (t0 >= t1) return;
    const bool on = j < N;
    const int64_t col = (int64_t)head * N + j;
    float* S_g = state + (int64_t)state_slots[s] * state_stride + (int64_t)head * N * N + (int64_t)j * N;
    float S[NMAX];
#pragma unroll
    for (int i = 0; i < NMAX; i++) S[i] = (on && i < N) ? S_g[i] : 0.f;
    const float w0j = on ? w0[col] : 0.f, uj = on ? u[col] : 0.f;

    // a row's r, k, z, v are loaded into registers while the row before it is summed, and
    // put into the other buffer after those sums: no load's latency stands between two rows
    float nr = 0.f, nk = 0.f, nz = 0.f, nv = 0.f;
    auto fetch = [&](int t) {
        if (on) {
            nr = r[(int64_t)t * r_stride + col];
            nk = k[(int64_t)t * k_stride + col];
            nz = z[(int64_t)t * z_stride + col];
            nv = v[(int64_t)t * v_stride + col];
        }
    };
    auto put = [&](int buf) {
        if (on) {
            sh[buf][0][j] = nr;
            sh[buf][1][j] = nk;
            sh[buf][2][j] = expf(-expf(nz + w0j));
            sh[buf][3][j] = uj * nk;
        }
    };
    fetch(t0);
    put(0);
    float vj = nv;
    if (t0 + 1 < t1) fetch(t0 + 1);
    __syncthreads();
    for (int t = t0; t < t1; t++) {
        const int buf = (t - t0) & 1;
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < NMAX; i++) {
            if (i < N) {
                const float a = sh[buf][1][i] * vj;
                acc += sh[buf][0][i] * (S[i] + sh[buf][3][i] * vj);
                S[i] = sh[buf][2][i] * S[i] + a;
            }
        }
        if (on) o[(int64_t)t * o_stride + col] = acc;
        if (t + 1 < t1) {
            put(buf ^ 1);
            vj = nv;
            if (t + 2 < t1) fetch(t + 2);
        }
        __syncthreads();
    }
    if (on) {
#pragma unroll
        for (int i = 0; i < NMAX; i++)
            if (i < N) S_g[i] = S[i];
    }
}

// Heads of N = 4 * IG channels, IG a power of two up to 32.  A CTA has JB value channels j0 ..
// j0 + JB - 1 of one head and (JB / JT) * IG threads; thread tid has g = tid % IG (key channels
// 4g .. 4g + 3) and JT value channels j0 + tid / IG + q * (JB / JT): what it reads of a row's
// (r, k, w, u k) from shared memory serves JT value channels, and shared-memory bandwidth is what
// bounds this kernel.  Rows are staged TS at a time: a batch's r, k, z, v are loaded into
// registers one whole batch of sums before they are needed, turned into (r, k, w, u * k) and
// put into the other shared-memory buffer after the sums of the batch in between, so that no
// load's latency stands between two rows.
// JT = 1 (many threads, short chains per row) is the faster form while the CTAs are few enough
// to be resident together, JT = 4 once they queue; a value channel's additions are the same in
// both, so the choice changes no bit of the result.
template <int IG, int JT_> struct WkvSplit {
    static constexpr int N = 4 * IG;
    static constexpr int JB = N < 256 / IG ? N : 256 / IG;
    static constexpr int JT = JT_;
    static constexpr int NTHR = JB / JT * IG;
    static constexpr int TS = (JT == 1 && N <= 64) ? 16 : 8;
};

template <int IG, int JT_>
__global__ void __launch_bounds__(WkvSplit<IG, JT_>::NTHR, JT_ == 1 ? 2 : 1)
wkv_scan_split_kernel(float* __restrict__ o, int64_t o_stride, const float* __restrict__ r, int64_t r_stride,
                      const float* __restrict__ k, int64_t k_stride, const float* __restrict__ v, int64_t v_stride,
                      const float* __restrict__ z, int64_t z_stride, const float* __restrict__ w0,
                      const float* __restrict__ u, float* __restrict__ state, int64_t state_stride,
                      const int* __restrict__ q_start, const int* __restrict__ state_slots) {
    using C = WkvSplit<IG, JT_>;
    constexpr int N = C::N, JB = C::JB, JT = C::JT, NTHR = C::NTHR, TS = C::TS, JQ = JB / JT;
    constexpr int ITEMS = (TS * N + NTHR - 1) / NTHR;       // (row, key channel) pairs a thread stages
    constexpr int VITEMS = (TS * JB + NTHR - 1) / NTHR;
    __shared__ float4 sh[2][TS][N];                         // (r, k, w, u * k) of key channel i at [(i % 4) * IG + i / 4]:
                                                            // the lanes of a value channel read neighbouring entries
    __shared__ float shv[2][TS][JB];
    griddep_wait();
    griddep_launch();
    constexpr int jsplit = N / JB;
    const int head = blockIdx.x / jsplit, j0 = (blockIdx.x - head * jsplit) * JB, s = blockIdx.y;
    const int t0 = q_start[s], t1 = q_start[s + 1];
    if (t0 >= t1) return;
    const int tid = threadIdx.x, g = tid % IG, jq = tid / IG;
    const int64_t base = (int64_t)head * N;
    float* S_base = state + (int64_t)state_slots[s] * state_stride + (base + j0 + jq) * N + 4 * g;
    float S[JT][4];
#pragma unroll
    for (int q = 0; q < JT; q++) {
        const float4 S4 = *reinterpret_cast<const float4*>(S_base + (int64_t)q * JQ * N);
        S[q][0] = S4.x; S[q][1] = S4.y; S[q][2] = S4.z; S[q][3] = S4.w;
    }

    float rr[ITEMS], rk[ITEMS], rz[ITEMS], rv[VITEMS];
    auto fetch = [&](int tb) {
#pragma unroll
        for (int e = 0; e < ITEMS; e++) {
            const int item = tid + e * NTHR, tt = item / N, i = item - tt * N, t = tb + tt;
            if (item < TS * N && t < t1) {
                rr[e] = r[(int64_t)t * r_stride + base + i];
                rk[e] = k[(int64_t)t * k_stride + base + i];
                rz[e] = z[(int64_t)t * z_stride + base + i];
            }
        }
#pragma unroll
        for (int e = 0; e < VITEMS; e++) {
            const int item = tid + e * NTHR, tt = item / JB, jj = item - tt * JB, t = tb + tt;
            if (item < TS * JB && t < t1) rv[e] = v[(int64_t)t * v_stride + base + j0 + jj];
        }
    };
    auto put = [&](int tb, int buf) {
#pragma unroll
        for (int e = 0; e < ITEMS; e++) {
            const int item = tid + e * NTHR, tt = item / N, i = item - tt * N, t = tb + tt;
            if (item < TS * N && t < t1)
                sh[buf][tt][(i & 3) * IG + (i >> 2)] =
                    make_float4(rr[e], rk[e], expf(-expf(rz[e] + w0[base + i])), u[base + i] * rk[e]);
        }
#pragma unroll
        for (int e = 0; e < VITEMS; e++) {
            const int item = tid + e * NTHR, tt = item / JB, jj = item - tt * JB, t = tb + tt;
            if (item < TS * JB && t < t1) shv[buf][tt][jj] = rv[e];
        }
    };
    fetch(t0);
    put(t0, 0);
    if (t0 + TS < t1) fetch(t0 + TS);
    __syncthreads();
    for (int tb = t0; tb < t1; tb += TS) {
        const int buf = ((tb - t0) / TS) & 1;
        // one row: the thread's parts of o for its JT value channels; the order of a value
        // channel's additions (key channels 4g .. 4g + 3, then the lanes' tree) is fixed
        auto sums = [&](int tt, float (&acc)[JT]) {
            float vj[JT];
#pragma unroll
            for (int q = 0; q < JT; q++) {
                vj[q] = shv[buf][tt][jq + q * JQ];
                acc[q] = 0.f;
            }
#pragma unroll
            for (int ii = 0; ii < 4; ii++) {
                const float4 c = sh[buf][tt][ii * IG + g];  // r, k, w, u * k of key channel 4g + ii
#pragma unroll
                for (int q = 0; q < JT; q++) {
                    const float a = c.y * vj[q];
                    acc[q] = fmaf(c.x, fmaf(c.w, vj[q], S[q][ii]), acc[q]);
                    S[q][ii] = fmaf(c.z, S[q][ii], a);
                }
            }
        };
        constexpr int RG = JT >= 4 ? 1 : 4 / JT;            // rows whose lane sums are formed together
        auto rows = [&](int tt, int n_rows) {
            float acc[RG][JT];
#pragma unroll
            for (int p = 0; p < RG; p++)
                if (p < n_rows) sums(tt + p, acc[p]);
#pragma unroll
            for (int off = IG / 2; off > 0; off >>= 1)
#pragma unroll
                for (int p = 0; p < RG; p++)
#pragma unroll
                    for (int q = 0; q < JT; q++) acc[p][q] += __shfl_xor_sync(0xffffffffu, acc[p][q], off);
            if (g == 0) {
#pragma unroll
                for (int p = 0; p < RG; p++)
#pragma unroll
                    for (int q = 0; q < JT; q++)
                        if (p < n_rows) o[(int64_t)(tb + tt + p) * o_stride + base + j0 + jq + q * JQ] = acc[p][q];
            }
        };
        if (tb + TS <= t1) {
            // a whole batch: no branch between the rows, so that their loads and shuffles overlap
#pragma unroll
            for (int tt = 0; tt < TS; tt += RG) rows(tt, RG);
        } else {
            for (int tt = 0; tb + tt < t1; tt += RG) rows(tt, min(RG, t1 - tb - tt));
        }
        if (tb + TS < t1) {
            put(tb + TS, buf ^ 1);                          // fetched while the batch before this one ran
            if (tb + 2 * TS < t1) fetch(tb + 2 * TS);
        }
        __syncthreads();
    }
#pragma unroll
    for (int q = 0; q < JT; q++)
        *reinterpret_cast<float4*>(S_base + (int64_t)q * JQ * N) = make_float4(S[q][0], S[q][1], S[q][2], S[q][3]);
}

// ---- the decay's outer product: z[t, a] = sum_r tanh(low[t, r]) * W2[a, r] ---------------------
// The inner width R is a handful (the decay's rank), far below what a matrix-product library is
// made for: tanh(low) of a few rows in shared memory, float32 sums in the order r = 0 .. R-1.
// A CTA has 256 channels a and up to DROWS rows t; a thread keeps eight weights of its channel
// in registers at a time and serves all the CTA's rows with them.
constexpr int DROWS = 16;

template <typename T>
__global__ void __launch_bounds__(256)
decay_outer_kernel(float* __restrict__ z, const float* __restrict__ low, int64_t low_stride, const T* __restrict__ w2,
                   int n, int A, int R) {
    extern __shared__ float th[];             // [DROWS][RP], RP = R rounded up to 8, zeros beyond R and beyond the rows
    griddep_wait();
    griddep_launch();
    const int RP = (R + 7) & ~7;
    const int t0 = blockIdx.y * DROWS, nt = min(DROWS, n - t0);
    for (int i = threadIdx.x; i < DROWS * RP; i += blockDim.x) {
        const int t = i / RP, r = i - t * RP;
        th[i] = (t < nt && r < R) ? tanhf(low[(int64_t)(t0 + t) * low_stride + r]) : 0.f;
    }
    __syncthreads();
    const int a = blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= A) return;
    const T* wr = w2 + (int64_t)a * R;
    float acc[DROWS];
#pragma unroll
    for (int t = 0; t < DROWS; t++) acc[t] = 0.f;
    for (int r0 = 0; r0 < RP; r0 += 8) {
        float w[8];
#pragma unroll
        for (int q = 0; q < 8; q++) w[q] = r0 + q < R ? to_f32(wr[r0 + q]) : 0.f;
#pragma unroll
        for (int t = 0; t < DROWS; t++)
#pragma unroll
            for (int q = 0; q < 8; q++) acc[t] += th[t * RP + r0 + q] * w[q];
    }
    for (int t = 0; t < nt; t++) z[(int64_t)(t0 + t) * A + a] = acc[t];
}

// ---- output: unit norm per head, gain, gate ---------------------------------------------
// one warp per (token, head); lane l adds the squares of its channels l, l + 32, ... in that
// order, then the lanes in a fixed tree.
template <typename T>
__global__ void __launch_bounds__(256)
gate_norm_kernel(T* __restrict__ y, const float* __restrict__ o, int64_t o_stride, const float* __restrict__ g,
                 int64_t g_stride, const float* __restrict__ gain, int64_t rows, int heads, int N, float eps) {
    griddep_wait();
    griddep_launch();
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int64_t t = row / heads;
    const int head = (int)(row - t * heads);
    const float* orow = o + t * o_stride + (int64_t)head * N;
    const float* grow = g + t * g_stride + (int64_t)head * N;
    float ss = 0.f;
    for (int c = lane; c < N; c += 32) ss += orow[c] * orow[c];
    ss = warp_sum(ss);
    const float scale = rsqrtf(ss / (float)N + eps);
    T* yrow = y + (t * heads + head) * N;
    for (int c = lane; c < N; c += 32) {
        const float gv = grow[c];
        yrow[c] = from_f32<T>(orow[c] * scale * gain[(int64_t)head * N + c] * (gv / (1.f + expf(-gv))));
    }
}

}  // namespace

// out [n_mix][n][d] and h [n][d] in the element type `dtype`; mu float32 [n_mix][d]; the previous
// row of request s lives at state[state_slots[s] * state_stride + prev_off .. + d].
extern "C" int kllm_wkv_shift_mix(void* out, const void* h, const float* mu, float* state, int64_t state_stride,
                                  int64_t prev_off, const int* q_start, const int* token_req, const int* state_slots,
                                  int n, int d, int n_mix, int dtype, void* stream) {
    if (n <= 0) return 0;
    if (d <= 0 || n_mix <= 0) KLLM_FAIL("wkv shift: width %d, %d mixes", d, n_mix);
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 1024 ? 256 : 128;
    if (dtype == KLLM_F32)
        kllm_launch((shift_mix_kernel<float>), dim3(n), dim3(threads), 0, s, (float*)out, (const float*)h, mu, state,
                    state_stride, prev_off, q_start, token_req, state_slots, n, d, n_mix);
    else if (dtype == KLLM_BF16)
        kllm_launch((shift_mix_kernel<bf16>), dim3(n), dim3(threads), 0, s, (bf16*)out, (const bf16*)h, mu, state,
                    state_stride, prev_off, q_start, token_req, state_slots, n, d, n_mix);
    else
        KLLM_FAIL("wkv shift: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}

// o, r, k, v, z float32 with `heads * N` dense columns and their own row strides; w0, u float32
// [heads * N]; n_rows rows in all; the state of request s is state[state_slots[s] * state_stride ..], [heads][N values][N keys].
extern "C" int kllm_wkv_scan(float* o, int64_t o_stride, const float* r, int64_t r_stride, const float* k,
                             int64_t k_stride, const float* v, int64_t v_stride, const float* z, int64_t z_stride,
                             const float* w0, const float* u, float* state, int64_t state_stride, const int* q_start,
                             const int* state_slots, int n_rows, int n_requests, int heads, int N, void* stream) {
    if (n_requests <= 0) return 0;
    if (heads <= 0 || N <= 0 || N > 128) KLLM_FAIL("wkv scan: %d heads of size %d (a head holds up to 128 channels)", heads, N);
    if (n_requests > 65535) KLLM_FAIL("wkv scan: %d requests in one launch", n_requests);
    cudaStream_t s = (cudaStream_t)stream;
    // Over prompts it is not started early: the scan's few, long-running CTAs would be placed on
    // whatever SMs the kernel before it has left free, two to an SM and others none, and run at
    // that imbalance to their end (measured: 0.1 ms a layer over a 2048-row prompt).  Steps of
    // a few rows per request (decode) gain from the early start like every short kernel.
    const bool early = n_rows <= 4 * n_requests;
#define KLLM_WKV_SPLIT_JT(IG, JT)                                                                                      \
    {                                                                                                                  \
        using C = WkvSplit<IG, JT>;                                                                                    \
        kllm_launch_dep(early, (wkv_scan_split_kernel<IG, JT>), dim3(heads * (C::N / C::JB), n_requests), dim3(C::NTHR), 0, s, o, \
                    o_stride, r, r_stride, k, k_stride, v, v_stride, z, z_stride, w0, u, state, state_stride, q_start, \
                    state_slots);                                                                                      \
        KLLM_LAUNCH_STATUS();                                                                                          \
    }
#define KLLM_WKV_SPLIT(IG)                                                                                             \
    if (N == 4 * IG) {                                                                                                 \
        constexpr int JB = WkvSplit<IG, 1>::JB;                                                                        \
        if (JB * IG < 256 || (int64_t)heads * (4 * IG / JB) * n_requests <= 2 * 148) KLLM_WKV_SPLIT_JT(IG, 1)           \
        KLLM_WKV_SPLIT_JT(IG, (JB * IG >= 256 ? 4 : 1))                                                                \
    }
    if (state_stride % 4 == 0 && ((uintptr_t)state & 15) == 0) {
        KLLM_WKV_SPLIT(4) KLLM_WKV_SPLIT(8) KLLM_WKV_SPLIT(16) KLLM_WKV_SPLIT(32)
    }
#undef KLLM_WKV_SPLIT_JT
#undef KLLM_WKV_SPLIT
#define KLLM_WKV(NMAX)                                                                                                  \
    kllm_launch_dep(early, (wkv_scan_kernel<NMAX>), dim3(heads, n_requests), dim3(NMAX), 0, s, o, o_stride, r, r_stride, k, k_stride, \
                v, v_stride, z, z_stride, w0, u, state, state_stride, q_start, state_slots, N)
    if (N <= 32) KLLM_WKV(32);
    else if (N <= 64) KLLM_WKV(64);
    else if (N <= 96) KLLM_WKV(96);
    else KLLM_WKV(128);
#undef KLLM_WKV
    KLLM_LAUNCH_STATUS();
}

// z float32 [n][A] contiguous; low float32 [n][R] at row stride low_stride; w2 [A][R] contiguous in
// the element type `dtype`.
extern "C" int kllm_wkv_decay_outer(float* z, const float* low, int64_t low_stride, const void* w2, int n, int A, int R,
                                    int dtype, void* stream) {
    if (n <= 0) return 0;
    if (A <= 0 || R <= 0) KLLM_FAIL("wkv decay: %d channels of rank %d", A, R);
    cudaStream_t s = (cudaStream_t)stream;
    const int row_tiles = (n + DROWS - 1) / DROWS;
    if (row_tiles > 65535) KLLM_FAIL("wkv decay: %d rows in one launch", n);
    const dim3 grid((A + 255) / 256, row_tiles);
    const size_t smem = (size_t)DROWS * ((R + 7) & ~7) * sizeof(float);
    if (smem > 48 * 1024) KLLM_FAIL("wkv decay: rank %d is beyond this kernel (use a matrix product)", R);
    if (dtype == KLLM_F32)
        kllm_launch((decay_outer_kernel<float>), grid, dim3(256), smem, s, z, low, low_stride, (const float*)w2, n, A, R);
    else if (dtype == KLLM_BF16)
        kllm_launch((decay_outer_kernel<bf16>), grid, dim3(256), smem, s, z, low, low_stride, (const bf16*)w2, n, A, R);
    else
        KLLM_FAIL("wkv decay: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}

// y [n][heads * N] contiguous in the element type `dtype`; o and g (the gate before its
// activation) float32 with their own row strides; gain float32 [heads * N].
extern "C" int kllm_wkv_gate_norm(void* y, const float* o, int64_t o_stride, const float* g, int64_t g_stride,
                                  const float* gain, int n, int heads, int N, float eps, int dtype, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t rows = (int64_t)n * heads;
    const dim3 grid((unsigned)((rows + 7) / 8));
    if (dtype == KLLM_F32)
        kllm_launch((gate_norm_kernel<float>), grid, dim3(256), 0, s, (float*)y, o, o_stride, g, g_stride, gain, rows, heads, N, eps);
    else if (dtype == KLLM_BF16)
        kllm_launch((gate_norm_kernel<bf16>), grid, dim3(256), 0, s, (bf16*)y, o, o_stride, g, g_stride, gain, rows, heads, N, eps);
    else
        KLLM_FAIL("wkv gate: unknown element type %d", dtype);
    KLLM_LAUNCH_STATUS();
}
