// Short causal convolution over time on the channels of a fused projection, with what follows it in a mixer
// that normalises queries, keys and values: bias, convolution, RMS norm of all query channels (and of all key
// channels) with a gain per channel, norm of each value head without a gain, and the store of keys and values
// into the paged cache.  One kernel per step and layer; a second, tiny one moves every request's last
// `taps - 1` projected rows into its convolution state.
//
//   x[t, c] = u[t, c] + bias[c]
//   y[t, c] = sum_j w[c, j] * x[t - taps + 1 + j, c]      rows before the step's first come from the request's
//                                                         state (zero for a new request)
// The state is float32 and holds x itself, so a row computed from the state equals the row computed from the
// step's own tokens bit for bit: how a prompt was cut into steps does not show.
#include "common.cuh"

namespace {

constexpr int kMaxTaps = 8;

__device__ __forceinline__ void load2(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x;
    b = v.y;
}
__device__ __forceinline__ void load2(const __nv_bfloat16* p, float& a, float& b) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    a = v.x;
    b = v.y;
}

// TAPS > 0: the number of taps is known when compiling (the loops over taps unroll to exactly that many); 0: any number.
template <typename T, int TAPS>
__global__ void __launch_bounds__(256)
conv_norm_store_kernel(const T* __restrict__ u, const float* __restrict__ bias, const float* __restrict__ taps_w, int taps_any,
                       const float* __restrict__ q_gain, const float* __restrict__ k_gain,
                       const float* __restrict__ state, const int* __restrict__ state_slots,
                       const int* __restrict__ token_request, const int* __restrict__ cu_seqlens,
                       T* __restrict__ q_out, T* __restrict__ cache, const int* __restrict__ slots,
                       long long page_stride, int page_size, int heads, int kv_heads, int dim, int vdim,
                       int channels, float eps) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float y[];  // channels floats
    __shared__ float red[32];
    const int taps = TAPS > 0 ? TAPS : taps_any;
    constexpr int kUnroll = TAPS > 0 ? TAPS : kMaxTaps;
    const int t = blockIdx.x;
    const int b = token_request[t];
    const int local = t - cu_seqlens[b];
    const int back = taps - 1;
    const float* st = state ? state + (size_t)state_slots[b] * back * channels : nullptr;
    const int cq = heads * dim, ck = cache ? kv_heads * dim : 0;
    float ssq = 0.f, ssk = 0.f;
    if (channels % 2 == 0 && cq % 2 == 0 && ck % 2 == 0) {
        // two neighbouring channels per thread and load; the taps' loads of a pair are all asked for before the first is used
        for (int c = 2 * threadIdx.x; c < channels; c += 2 * blockDim.x) {
            const float b0 = bias ? bias[c] : 0.f, b1 = bias ? bias[c + 1] : 0.f;
            float x0[kUnroll], x1[kUnroll];
#pragma unroll
            for (int j = 0; j < kUnroll; ++j) {
                if (j < taps) {
                    const int src = local - (back - j);
                    if (src >= 0) {
                        load2(u + (size_t)(t - (back - j)) * channels + c, x0[j], x1[j]);
                        x0[j] += b0;
                        x1[j] += b1;
                    } else {
                        const float2 v = *reinterpret_cast<const float2*>(st + (size_t)(back + src) * channels + c);
                        x0[j] = v.x;
                        x1[j] = v.y;
                    }
                }
            }
            float a0 = 0.f, a1 = 0.f;
            if (taps_w) {
#pragma unroll
                for (int j = 0; j < kUnroll; ++j) {
                    if (j < taps) {
                        a0 = fmaf(taps_w[(size_t)c * taps + j], x0[j], a0);
                        a1 = fmaf(taps_w[(size_t)(c + 1) * taps + j], x1[j], a1);
                    }
                }
            } else {
                a0 = x0[0];
                a1 = x1[0];
            }
            y[c] = a0;
            y[c + 1] = a1;
            if (c < cq) ssq += a0 * a0 + a1 * a1;
            else if (c < cq + ck) ssk += a0 * a0 + a1 * a1;
        }
    } else {
        for (int c = threadIdx.x; c < channels; c += blockDim.x) {
            const float bc = bias ? bias[c] : 0.f;
            float acc = 0.f;
            if (taps_w) {
                for (int j = 0; j < taps; ++j) {
                    const int src = local - (back - j);
                    const float x = src >= 0 ? to_f32(u[(size_t)(t - (back - j)) * channels + c]) + bc
                                             : st[(size_t)(back + src) * channels + c];
                    acc = fmaf(taps_w[(size_t)c * taps + j], x, acc);
                }
            } else {
                acc = to_f32(u[(size_t)t * channels + c]) + bc;
            }
            y[c] = acc;
            if (c < cq) ssq += acc * acc;
            else if (c < cq + ck) ssk += acc * acc;
        }
    }
    const float tq = block_sum(ssq, red);
    const float inv_q = 1.0f / sqrtf(tq / (float)cq + eps);
    for (int c = threadIdx.x; c < cq; c += blockDim.x)
        q_out[(size_t)t * cq + c] = from_f32<T>(y[c] * inv_q * q_gain[c]);
    if (!cache) return;
    const float tk = block_sum(ssk, red);
    const float inv_k = 1.0f / sqrtf(tk / (float)ck + eps);
    const int slot = slots[t];
    const int page = slot / page_size, off = slot % page_size;
    T* kp = cache + (size_t)page * page_stride;
    T* vp = kp + (size_t)kv_heads * page_size * dim;
    for (int c = threadIdx.x; c < ck; c += blockDim.x) {
        const int g = c / dim, d = c % dim;
        kp[((size_t)g * page_size + off) * dim + d] = from_f32<T>(y[cq + c] * inv_k * k_gain[c]);
    }
    // each value head divided by its own root mean square: a warp per head
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    const float* yv = y + cq + ck;
    for (int g = warp; g < kv_heads; g += nwarp) {
        float ss = 0.f;
        for (int d = lane; d < vdim; d += 32) ss += yv[g * vdim + d] * yv[g * vdim + d];
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
        for (int d = lane; d < vdim; d += 32)
            vp[((size_t)g * page_size + off) * vdim + d] = from_f32<T>(yv[g * vdim + d] * inv);
    }
}

// The last `taps - 1` rows of x of every request become its state (older state rows move up when the step
// brought fewer).  One block per request; a thread owns a channel, reads all it needs, then writes.
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_kernel(const T* __restrict__ u, const float* __restrict__ bias, int taps, float* __restrict__ state,
                  const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens, int channels) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const int first = cu_seqlens[b], n = cu_seqlens[b + 1] - first;
    const int back = taps - 1;
    float* st = state + (size_t)state_slots[b] * back * channels;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
        const float bc = bias ? bias[c] : 0.f;
        float keep[kMaxTaps];
#pragma unroll
        for (int r = 0; r < kMaxTaps - 1; ++r) {
            if (r < back) {
                const int src = n - back + r;
                keep[r] = src >= 0 ? to_f32(u[(size_t)(first + src) * channels + c]) + bc : st[(size_t)(back + src) * channels + c];
            }
        }
#pragma unroll
        for (int r = 0; r < kMaxTaps - 1; ++r)
            if (r < back) st[(size_t)r * channels + c] = keep[r];
    }
}

}  // namespace

// u [tokens, channels]: query channels (heads * dim), then, when `cache` is given, key channels (kv_heads * dim)
// and value channels (kv_heads * vdim).  bias, taps_w [channels, taps], gains: float32 (bias and taps_w may be
// null: no bias, one tap).  state [slots, taps - 1, channels] float32 (null with one tap).  q_out [tokens, heads * dim].
// cache: pages of `page_stride` elements, key plane [kv_heads, page_size, dim] then value plane [kv_heads, page_size, vdim].
LLM_API int llm_conv_norm_store(const void* u, const float* bias, const float* taps_w, int taps, const float* q_gain,
                                const float* k_gain, float* state, const int* state_slots, const int* token_request,
                                const int* cu_seqlens, void* q_out, void* cache, const int* slots, long long page_stride,
                                int page_size, int dtype, int tokens, int requests, int heads, int kv_heads, int dim,
                                int vdim, float eps, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (taps < 1 || taps > kMaxTaps) LLM_FAIL(-1, "short convolution: %d taps are not supported (1 to %d)", taps, kMaxTaps);
    if (taps > 1 && (!state || !taps_w)) LLM_FAIL(-1, "short convolution: %d taps need weights and a state", taps);
    if (!taps_w) taps = 1;
    const int channels = heads * dim + (cache ? kv_heads * (dim + vdim) : 0);
    const size_t smem = (size_t)channels * sizeof(float);
    if (smem > 200 * 1024) LLM_FAIL(-1, "short convolution: %d channels do not fit shared memory", channels);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
#define LLM_CONV(TT)                                                                                                       \
    do {                                                                                                                   \
        if (smem > 48 * 1024)                                                                                              \
            cudaFuncSetAttribute(conv_norm_store_kernel<T, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        llm_launch(conv_norm_store_kernel<T, TT>, tokens, 256, smem, stream, (const T*)u, bias, taps_w, taps, q_gain, k_gain, \
                   (const float*)state, state_slots, token_request, cu_seqlens, (T*)q_out, (T*)cache, slots, page_stride,   \
                   page_size, heads, kv_heads, dim, vdim, channels, eps);                                                   \
    } while (0)
        switch (taps) {           // the usual sizes unrolled, the rest by the general form
            case 1: LLM_CONV(1); break;
            case 2: LLM_CONV(2); break;
            case 3: LLM_CONV(3); break;
            case 4: LLM_CONV(4); break;
            default: LLM_CONV(0); break;
        }
#undef LLM_CONV
        LLM_CHECK_LAUNCH("conv_norm_store");
        if (taps > 1) {
            const int by = (channels + 255) / 256 < 8 ? (channels + 255) / 256 : 8;
            llm_launch(conv_state_kernel<T>, dim3(requests, by), 256, 0, stream, (const T*)u, bias, taps, state,
                       state_slots, cu_seqlens, channels);
            LLM_CHECK_LAUNCH("conv_state");
        }
        return 0;
    });
}

LLM_TRACE_EXPORT(short_conv)
