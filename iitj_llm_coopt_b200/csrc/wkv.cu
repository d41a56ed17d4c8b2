// The wkv mixer: a matrix state per head with a decay per key channel that each token chooses.
//
// llm_token_shift:  m_s[t] = x[t] + (x'[t] - x[t]) * mu_s for every stream s, x' the row before (for a request's first row of
//                   the step: the row its state slot holds; zero for a new request).  out [streams * T, width].
// llm_wkv_decay:    w[t, c] = exp(-exp(W2[c, :] . tanh(low[t, :]) + w0[c])), all float32.
// llm_wkv_scan:     per (request, head), token by token in order:
//                       o_t[j] = sum_i r_t[i] * (S[i][j] + u[i] * k_t[i] * v_t[j]);   S[i][j] = w_t[i] * S[i][j] + k_t[i] * v_t[j]
//                   then each head's o divided by its root mean square, times gain, times silu(g).  S [head_dim (key i),
//                   head_dim (value j)] float32 is read from and left in the request's state slot; four threads share column j
//                   (a quarter of its rows each, in registers; their sums meet by two shuffles).  Sixteen tokens' r, k, v, g, w rows
//                   (eight at head sizes above 64) are staged in shared memory at a time, asked for while the rows before them
//                   are walked, and read as 16-byte pieces; the head norm of those tokens runs after their walk, a warp per token.  The walk is strictly sequential in one order, so
//                   how a prompt was cut into steps does not change a single bit.  With `x` and `before` the request's last row
//                   of the step becomes the row its next step shifts in.
#include "common.cuh"

namespace {

constexpr int kChunk = 16;

template <typename T>
__global__ void __launch_bounds__(256)
token_shift_kernel(const T* __restrict__ x, const float* __restrict__ mu, const float* __restrict__ before,
                   const int* __restrict__ state_slots, const int* __restrict__ token_request, const int* __restrict__ cu_seqlens,
                   T* __restrict__ out, int tokens, int width, int streams) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = token_request[t];
    const bool first = t == cu_seqlens[b];
    const float* prev_state = before + (size_t)state_slots[b] * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = to_f32(x[(size_t)t * width + c]);
        const float p = first ? prev_state[c] : to_f32(x[(size_t)(t - 1) * width + c]);
        for (int s = 0; s < streams; ++s)
            out[((size_t)s * tokens + t) * width + c] = from_f32<T>(v + (p - v) * mu[(size_t)s * width + c]);
    }
}

__global__ void __launch_bounds__(256)
wkv_decay_kernel(const float* __restrict__ low, const float* __restrict__ w2, const float* __restrict__ w0, float* __restrict__ out,
                 int channels, int rank) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float th[];
    const size_t t = blockIdx.x;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) th[j] = tanhf(low[t * rank + j]);
    __syncthreads();
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        const float* row = w2 + (size_t)c * rank;
        float acc = 0.f;
        for (int j = 0; j < rank; ++j) acc = fmaf(row[j], th[j], acc);
        out[t * channels + c] = expf(-expf(acc + w0[c]));
    }
}

template <typename T, int DMAX>
__global__ void __launch_bounds__(DMAX * 4)
wkv_scan_kernel(const T* __restrict__ rkvg, const float* __restrict__ decay, const float* __restrict__ u, const float* __restrict__ gain,
                float eps, float* __restrict__ state, const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens,
                T* __restrict__ out, int tokens, int heads, int dim, int write, const T* __restrict__ x, float* __restrict__ before,
                int width) {
    pdl_trigger();
    pdl_wait();
    // Four threads share a column j of S: thread (j, p) keeps the rows 16 q + 4 p + (0..3), q = 0 .. DMAX / 16 - 1, so the four
    // read neighbouring 16-byte pieces of the staged rows (no bank conflict, and all columns read the same piece at once).
    constexpr int R = DMAX / 4, THREADS = DMAX * 4;
    constexpr int CH = DMAX > 64 ? kChunk / 2 : kChunk;          // tokens staged at a time
    constexpr int PER = CH * DMAX / THREADS;                     // elements of each staged array a thread brings
    __shared__ __align__(16) float sr[CH][DMAX], sk[CH][DMAX], sw[CH][DMAX], sv[CH][DMAX], sg[CH][DMAX], so[CH][DMAX];
    __shared__ __align__(16) float su[DMAX];
    const int b = blockIdx.x / heads, h = blockIdx.x % heads;
    const int lo = cu_seqlens[b], hi = cu_seqlens[b + 1];
    if (hi <= lo) return;
    const int tid = threadIdx.x, j = tid >> 2, p = tid & 3;
    const int n = heads * dim;
    float* S = state + ((size_t)state_slots[b] * heads + h) * dim * dim;
    float col[R];
#pragma unroll
    for (int q = 0; q < R / 4; ++q)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 16 * q + 4 * p + e;
            col[4 * q + e] = i < dim && j < dim ? S[(size_t)i * dim + j] : 0.f;
        }
    for (int i = tid; i < DMAX; i += THREADS) su[i] = i < dim ? u[(size_t)h * dim + i] : 0.f;
    const int warp = tid >> 5, lane = tid & 31, nwarp = THREADS >> 5;
    // A chunk's rows are asked for while the chunk before is walked (channels beyond dim are zero and stay out of every sum).
    float lr[PER], lk[PER], lv[PER], lg[PER], lw[PER];
    auto fetch = [&](int t0) {
        const int cnt = min(CH, hi - t0);
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int idx = tid + e * THREADS, c = idx / DMAX, i = idx % DMAX;
            const bool live = c < cnt && i < dim;
            const size_t row = (size_t)(t0 + c) * n + (size_t)h * dim + i, stream = (size_t)tokens * n;
            lr[e] = live ? to_f32(rkvg[row]) : 0.f;
            lk[e] = live ? to_f32(rkvg[row + stream]) : 0.f;
            lv[e] = live ? to_f32(rkvg[row + 2 * stream]) : 0.f;
            lg[e] = live ? to_f32(rkvg[row + 3 * stream]) : 0.f;
            lw[e] = live ? decay[(size_t)(t0 + c) * n + (size_t)h * dim + i] : 0.f;
        }
    };
    fetch(lo);
    for (int t0 = lo; t0 < hi; t0 += CH) {
        const int cnt = min(CH, hi - t0);
        __syncthreads();                                  // the norm phase of the chunk before is done with the staged rows
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            const int idx = tid + e * THREADS, c = idx / DMAX, i = idx % DMAX;
            sr[c][i] = lr[e]; sk[c][i] = lk[e]; sv[c][i] = lv[e]; sg[c][i] = lg[e]; sw[c][i] = lw[e];
        }
        __syncthreads();
        if (t0 + CH < hi) fetch(t0 + CH);
        for (int c = 0; c < cnt; ++c) {
            const float vj = sv[c][j];
            float o = 0.f;
#pragma unroll
            for (int q = 0; q < R / 4; ++q) {
                const int base = 16 * q + 4 * p;
                const float4 r4 = *reinterpret_cast<const float4*>(&sr[c][base]);
                const float4 k4 = *reinterpret_cast<const float4*>(&sk[c][base]);
                const float4 w4 = *reinterpret_cast<const float4*>(&sw[c][base]);
                const float4 u4 = *reinterpret_cast<const float4*>(&su[base]);
                float kv;
                kv = k4.x * vj; o = fmaf(r4.x, fmaf(u4.x, kv, col[4 * q]), o);     col[4 * q] = fmaf(w4.x, col[4 * q], kv);
                kv = k4.y * vj; o = fmaf(r4.y, fmaf(u4.y, kv, col[4 * q + 1]), o); col[4 * q + 1] = fmaf(w4.y, col[4 * q + 1], kv);
                kv = k4.z * vj; o = fmaf(r4.z, fmaf(u4.z, kv, col[4 * q + 2]), o); col[4 * q + 2] = fmaf(w4.z, col[4 * q + 2], kv);
                kv = k4.w * vj; o = fmaf(r4.w, fmaf(u4.w, kv, col[4 * q + 3]), o); col[4 * q + 3] = fmaf(w4.w, col[4 * q + 3], kv);
            }
            o += __shfl_xor_sync(0xffffffffu, o, 1);
            o += __shfl_xor_sync(0xffffffffu, o, 2);
            if (p == 0) so[c][j] = o;
        }
        __syncthreads();
        for (int c = warp; c < cnt; c += nwarp) {         // head norm, gain and gate: a warp per token
            float ss = 0.f;
            for (int i = lane; i < dim; i += 32) ss += so[c][i] * so[c][i];
            const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
            for (int i = lane; i < dim; i += 32) {
                const size_t ch = (size_t)h * dim + i;
                const float g = sg[c][i];
                out[(size_t)(t0 + c) * n + ch] = from_f32<T>(so[c][i] * inv * gain[ch] * (g / (1.0f + expf(-g))));
            }
        }
    }
    if (write && j < dim)
#pragma unroll
        for (int q = 0; q < R / 4; ++q)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = 16 * q + 4 * p + e;
                if (i < dim) S[(size_t)i * dim + j] = col[4 * q + e];
            }
    if (before && h == 0)
        for (int c = tid; c < width; c += THREADS) before[(size_t)state_slots[b] * width + c] = to_f32(x[(size_t)(hi - 1) * width + c]);
}

}  // namespace

LLM_API int llm_token_shift(const void* x, const float* mu, const float* before, const int* state_slots, const int* token_request,
                            const int* cu_seqlens, void* out, int dtype, int tokens, int width, int streams, cudaStream_t stream) {
    if (tokens == 0) return 0;
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(token_shift_kernel<T>, (unsigned)tokens, 256, 0, stream, (const T*)x, mu, before, state_slots, token_request,
                   cu_seqlens, (T*)out, tokens, width, streams);
        LLM_CHECK_LAUNCH("token_shift");
        return 0;
    });
}

LLM_API int llm_wkv_decay(const float* low, const float* w2, const float* w0, float* out, int tokens, int channels, int rank,
                          cudaStream_t stream) {
    if (tokens == 0) return 0;
    if ((size_t)rank * sizeof(float) > 48 * 1024) LLM_FAIL(-1, "wkv_decay: rank %d is too large", rank);
    llm_launch(wkv_decay_kernel, (unsigned)tokens, 256, (size_t)rank * sizeof(float), stream, low, w2, w0, out, channels, rank);
    LLM_CHECK_LAUNCH("wkv_decay");
    return 0;
}

// rkvg [4 * tokens, heads * dim] of `dtype` (the rows of r, then of k, v and g); decay [tokens, heads * dim] float32; state
// [slots, heads, dim, dim] float32.  x [tokens, width] and before [slots, width] (or null): the shifted-in row to leave behind.
LLM_API int llm_wkv_scan(const void* rkvg, const float* decay, const float* u, const float* gain, float eps, float* state,
                         const int* state_slots, const int* cu_seqlens, void* out, int dtype, int tokens, int requests, int heads,
                         int dim, int write, const void* x, float* before, int width, cudaStream_t stream) {
    if (requests == 0) return 0;
    if (dim <= 0 || dim > 128) LLM_FAIL(-1, "wkv_scan: head size %d must be in [1, 128]", dim);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        const unsigned blocks = (unsigned)requests * heads;
#define LLM_WKV_CASE(DMAX)                                                                                                   \
        llm_launch(wkv_scan_kernel<T, DMAX>, blocks, DMAX * 4, 0, stream, (const T*)rkvg, decay, u, gain, eps, state, state_slots,   \
                   cu_seqlens, (T*)out, tokens, heads, dim, write, (const T*)x, before, width)
        if (dim <= 32) LLM_WKV_CASE(32);
        else if (dim <= 64) LLM_WKV_CASE(64);
        else LLM_WKV_CASE(128);
#undef LLM_WKV_CASE
        LLM_CHECK_LAUNCH("wkv_scan");
        return 0;
    });
}

LLM_TRACE_EXPORT(wkv)
