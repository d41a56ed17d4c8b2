// Norms that sit on a branch's output, and the clamped gated activation.
//
// llm_norm_add:     residual[t] (+)= branch[t] * rsqrt(mean(branch[t]^2) + eps) * weight   (float32 statistics and sum),
//                   and optionally a copy of the new residual row in the engine's type, which the next sub-layer reads.
//                   One block per row, the row held in registers between the two passes, sums in a fixed order.
// llm_glu_clamped:  act = g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit),
//                   from one [T, 2 * inner] row of gate columns followed by up columns.
#include "common.cuh"

namespace {

constexpr int kNormThreads = 256;
constexpr int kNormPer = 8;          // elements a thread holds: rows up to 2048 * ... are walked in rounds of 2048

template <typename TB, typename TW, typename TC>
__global__ void __launch_bounds__(kNormThreads)
norm_add_kernel(float* __restrict__ residual, const TB* __restrict__ branch, const TW* __restrict__ weight,
                TC* __restrict__ cast, int width, float eps, int accumulate) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const TB* b = branch + row * width;
    float* res = residual + row * width;
    float ss = 0.f;
    float held[kNormPer];
    // first pass: sum of squares (the first kNormPer rounds of the row stay in registers)
#pragma unroll
    for (int j = 0; j < kNormPer; ++j) {
        const int i = threadIdx.x + j * kNormThreads;
        held[j] = i < width ? to_f32(b[i]) : 0.f;
        ss += held[j] * held[j];
    }
    for (int i = threadIdx.x + kNormPer * kNormThreads; i < width; i += kNormThreads) {
        const float v = to_f32(b[i]);
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
#pragma unroll
    for (int j = 0; j < kNormPer; ++j) {
        const int i = threadIdx.x + j * kNormThreads;
        if (i < width) {
            float y = held[j] * inv * to_f32(weight[i]);
            if (accumulate) y += res[i];
            res[i] = y;
            if (cast) cast[row * width + i] = from_f32<TC>(y);
        }
    }
    for (int i = threadIdx.x + kNormPer * kNormThreads; i < width; i += kNormThreads) {
        float y = to_f32(b[i]) * inv * to_f32(weight[i]);
        if (accumulate) y += res[i];
        res[i] = y;
        if (cast) cast[row * width + i] = from_f32<TC>(y);
    }
}

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ act, int tokens, int inner, float limit, float slope) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)tokens * inner;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inner, c = i % inner;
        const float g = fminf(to_f32(gu[t * 2 * inner + c]), limit);
        const float u = fminf(fmaxf(to_f32(gu[t * 2 * inner + inner + c]), -limit), limit);
        act[i] = from_f32<T>(g / (1.0f + expf(-slope * g)) * (u + 1.0f));
    }
}

}  // namespace

// branch [tokens, width] of `branch_dtype`; weight float32 or bfloat16 (`weight_dtype`); cast: null or [tokens, width] of
// `cast_dtype`.  accumulate == 0 writes the normed row instead of adding it (an embedding's norm).
LLM_API int llm_norm_add(float* residual, const void* branch, int branch_dtype, const void* weight, int weight_dtype,
                         void* cast, int cast_dtype, int tokens, int width, float eps, int accumulate, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (width <= 0) LLM_FAIL(-1, "norm_add: width %d", width);
    return llm_dispatch_dtype(branch_dtype, [&](auto tb) {
        using TB = decltype(tb);
        return llm_dispatch_dtype(weight_dtype, [&](auto tw) {
            using TW = decltype(tw);
            return llm_dispatch_dtype(cast ? cast_dtype : LLM_BF16, [&](auto tc) {
                using TC = decltype(tc);
                llm_launch(norm_add_kernel<TB, TW, TC>, (unsigned)tokens, kNormThreads, 0, stream, residual, (const TB*)branch,
                           (const TW*)weight, (TC*)cast, width, eps, accumulate);
                LLM_CHECK_LAUNCH("norm_add");
                return 0;
            });
        });
    });
}

LLM_API int llm_glu_clamped(const void* gu, void* act, int dtype, int tokens, int inner, float limit, float slope,
                            cudaStream_t stream) {
    if (tokens == 0 || inner == 0) return 0;
    const size_t n = (size_t)tokens * inner;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(glu_clamped_kernel<T>, blocks, 256, 0, stream, (const T*)gu, (T*)act, tokens, inner, limit, slope);
        LLM_CHECK_LAUNCH("glu_clamped");
        return 0;
    });
}

LLM_TRACE_EXPORT(branch_norm)
