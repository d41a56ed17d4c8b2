// Paged attention whose heads talk to each other before the softmax, general form (float32 arithmetic, any
// sizes): for a query at position i of a request and every key j it sees,
//     s[g, j] = scale * q[g] . k[kv(g), j] - slope[g] * (i - j)          all query heads g
//     a[h, j] = sum_g talk[h, g] * s[g, j]
//     p[h, :] = softmax_j a[h, :],     out[h] = sum_j p[h, j] v[kv(h), j]
// A query sees the keys j <= i of its request; with chunk > 0 only those of its own chunk (j / chunk == i / chunk,
// counted from the request's position 0).  Because every head's score of a key enters every head's softmax,
// one block works on all heads of a token: the scores of a tile of 32 keys land in shared memory, each warp mixes them
// for its own heads (a lane per key) and then runs the running softmax and the value sum of those heads.
//
// Key tiles start at multiples of 32 of the key position and sums run in a fixed order, so a position's result
// does not depend on how the request was cut into steps or on what else is in the batch.
//
// Cache layout: pages of `page_stride` elements; key plane [kv_heads, page_size, dim], then, `v_off` elements in,
// value plane [kv_heads, page_size, vdim].
#include "common.cuh"

namespace {

constexpr int kTile = 32;
constexpr int kMaxValueDim = 256;

template <typename T>
__device__ __forceinline__ float dot_any(const T* __restrict__ k, const float* __restrict__ q, int d, bool vec);

template <>
__device__ __forceinline__ float dot_any<float>(const float* __restrict__ k, const float* __restrict__ q, int d, bool vec) {
    float acc = 0.f;
    if (vec) {
        for (int i = 0; i < d; i += 4) {
            const float4 kv = *reinterpret_cast<const float4*>(k + i);
            const float4 qv = *reinterpret_cast<const float4*>(q + i);
            acc = fmaf(kv.x, qv.x, acc);
            acc = fmaf(kv.y, qv.y, acc);
            acc = fmaf(kv.z, qv.z, acc);
            acc = fmaf(kv.w, qv.w, acc);
        }
    } else {
        for (int i = 0; i < d; ++i) acc = fmaf(k[i], q[i], acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot_any<__nv_bfloat16>(const __nv_bfloat16* __restrict__ k, const float* __restrict__ q,
                                                         int d, bool vec) {
    float acc = 0.f;
    if (vec) {
        for (int i = 0; i < d; i += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
            const float4 qa = *reinterpret_cast<const float4*>(q + i), qb = *reinterpret_cast<const float4*>(q + i + 4);
            const float qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(p[j]);
                acc = fmaf(f.x, qv[2 * j], acc);
                acc = fmaf(f.y, qv[2 * j + 1], acc);
            }
        }
    } else {
        for (int i = 0; i < d; ++i) acc = fmaf(__bfloat162float(k[i]), q[i], acc);
    }
    return acc;
}

__device__ __forceinline__ float2 pair_f32(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 pair_f32(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename T, int HPW>
__global__ void talking_attn_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ cache, long long page_stride,
                                    long long v_off, const int* __restrict__ block_table, int table_width,
                                    const int* __restrict__ token_request, const int* __restrict__ positions,
                                    const float* __restrict__ talk, const float* __restrict__ slopes,
                                    T* __restrict__ out, int out_stride, int heads, int kv_heads, int dim, int vdim,
                                    int page_size, int chunk, float scale, int vec) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    const int hp = (heads + 7) & ~7;            // a row of the mixing matrix in shared memory, padded to 32 bytes
    float* qs = smem;                           // [heads, dim]
    float* talk_s = qs + ((heads * dim + 3) & ~3);   // [heads (g), hp (h)]: transposed, so that a warp's heads lie side by side
    float* S = talk_s + heads * hp;             // [heads, kTile] scores before mixing
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[t];
    const int lo = chunk > 0 ? (pos / chunk) * chunk : 0;
    const int* table = block_table + (size_t)token_request[t] * table_width;
    const int group = heads / kv_heads;

    for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) qs[i] = to_f32(q[(size_t)t * q_stride + i]);
    for (int i = threadIdx.x; i < heads * hp; i += blockDim.x) {
        const int g = i / hp, h = i % hp;
        talk_s[i] = h < heads ? talk[h * heads + g] : 0.f;
    }

    constexpr int kOwn = kMaxValueDim / 32;
    float acc[HPW][kOwn], m[HPW], l[HPW];
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int r = 0; r < kOwn; ++r) acc[i][r] = 0.f;
    }
    __syncthreads();

    for (int k0 = lo & ~(kTile - 1); k0 <= pos; k0 += kTile) {
        const int j = k0 + lane;
        const bool valid = j >= lo && j <= pos;
        long long page_base = 0;
        int off = 0;
        if (valid) {
            page_base = (long long)table[j / page_size] * page_stride;
            off = j % page_size;
        }
        // scores of all heads for the tile's keys: a warp takes one head at a time, a lane one key
        for (int g = warp; g < heads; g += (blockDim.x >> 5)) {
            float s = 0.f;
            if (valid) {
                const T* krow = cache + page_base + ((size_t)(g / group) * page_size + off) * dim;
                s = scale * dot_any<T>(krow, qs + g * dim, dim, vec != 0) - slopes[g] * (float)(pos - j);
            }
            S[g * kTile + lane] = s;
        }
        __syncthreads();
        // the warp's own heads after mixing: a[i] = sum_g talk[h_i, g] * s[g, this lane's key], g ascending
        float a[HPW];
#pragma unroll
        for (int i = 0; i < HPW; ++i) a[i] = 0.f;
        {
            const float* trow = talk_s + warp * HPW;
            for (int g = 0; g < heads; ++g, trow += hp) {
                const float sg = S[g * kTile + lane];
                if (HPW % 4 == 0) {
#pragma unroll
                    for (int i = 0; i < HPW; i += 4) {
                        const float4 w = *reinterpret_cast<const float4*>(trow + i);
                        a[i] = fmaf(w.x, sg, a[i]);
                        a[i + 1] = fmaf(w.y, sg, a[i + 1]);
                        a[i + 2] = fmaf(w.z, sg, a[i + 2]);
                        a[i + 3] = fmaf(w.w, sg, a[i + 3]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < HPW; ++i) a[i] = fmaf(trow[i], sg, a[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < HPW; ++i) {
            const int h = warp * HPW + i;
            if (h >= heads) break;                       // the whole warp leaves together
            const float s = valid ? a[i] : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(s));   // finite: every tile holds a visible key
            const float corr = expf(m[i] - m_new);          // 0 on the first tile
            const float p = valid ? expf(s - m_new) : 0.f;
            l[i] = l[i] * corr + warp_sum(p);
            m[i] = m_new;
#pragma unroll
            for (int r = 0; r < kOwn; ++r) acc[i][r] *= corr;
            const long long vo = page_base + v_off + ((long long)(h / group) * page_size + off) * vdim;
            // eight keys at a time: their value rows are all asked for before the first is used
            for (int j0 = 0; j0 < kTile; j0 += 8) {
                float pj[8];
                const T* v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    pj[u] = __shfl_sync(0xffffffffu, p, j0 + u);
                    v[u] = cache + __shfl_sync(0xffffffffu, vo, j0 + u);
                }
                if (pj[0] + pj[1] + pj[2] + pj[3] + pj[4] + pj[5] + pj[6] + pj[7] == 0.f) continue;   // same for the whole warp
                if (vec) {
                    // a lane owns the dims 2 * lane, 2 * lane + 1 (+ 64, + 128, ...): one load for two of them
#pragma unroll
                    for (int r = 0; r < kOwn; r += 2) {
                        const int d = 2 * lane + 32 * r;
                        if (d < vdim) {
                            float2 x[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) x[u] = pj[u] != 0.f ? pair_f32(v[u] + d) : make_float2(0.f, 0.f);
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                acc[i][r] = fmaf(pj[u], x[u].x, acc[i][r]);
                                acc[i][r + 1] = fmaf(pj[u], x[u].y, acc[i][r + 1]);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < kOwn; ++r) {
                        const int d = lane + 32 * r;
                        if (d < vdim) {
                            float x[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) x[u] = pj[u] != 0.f ? to_f32(v[u][d]) : 0.f;
#pragma unroll
                            for (int u = 0; u < 8; ++u) acc[i][r] = fmaf(pj[u], x[u], acc[i][r]);
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
        const int h = warp * HPW + i;
        if (h >= heads) break;
        const float inv = 1.0f / l[i];
        T* orow = out + (size_t)t * out_stride + (size_t)h * vdim;
        if (vec) {
#pragma unroll
            for (int r = 0; r < kOwn; r += 2) {
                const int d = 2 * lane + 32 * r;
                if (d < vdim) store_pair(orow + d, acc[i][r] * inv, acc[i][r + 1] * inv);
            }
        } else {
#pragma unroll
            for (int r = 0; r < kOwn; ++r) {
                const int d = lane + 32 * r;
                if (d < vdim) orow[d] = from_f32<T>(acc[i][r] * inv);
            }
        }
    }
}

template <typename T, int HPW>
int launch_talking(const void* q, int q_stride, const void* cache, long long page_stride, long long v_off,
                   const int* block_table, int table_width, const int* token_request, const int* positions,
                   const float* talk, const float* slopes, void* out, int out_stride, int tokens, int heads, int kv_heads,
                   int dim, int vdim, int page_size, int chunk, float scale, int vec, cudaStream_t stream) {
    const int warps = (heads + HPW - 1) / HPW;
    const size_t smem = sizeof(float) * ((((size_t)heads * dim + 3) & ~(size_t)3) + (size_t)heads * ((heads + 7) & ~7) + (size_t)heads * kTile);
    if (smem > 200 * 1024) LLM_FAIL(-1, "talking attention: %d heads of %d dims do not fit shared memory", heads, dim);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(talking_attn_kernel<T, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    llm_launch(talking_attn_kernel<T, HPW>, tokens, warps * 32, smem, stream, (const T*)q, q_stride, (const T*)cache,
               page_stride, v_off, block_table, table_width, token_request, positions, talk, slopes, (T*)out, out_stride,
               heads, kv_heads, dim, vdim, page_size, chunk, scale, vec);
    LLM_CHECK_LAUNCH("talking_attention");
    return 0;
}

}  // namespace

LLM_API int llm_talking_attention(const void* q, int q_stride, const void* cache, long long page_stride, long long v_off,
                                  const int* block_table, int table_width, const int* token_request,
                                  const int* positions, const float* talk, const float* slopes, void* out,
                                  int out_stride, int dtype, int tokens, int heads, int kv_heads, int dim, int vdim,
                                  int page_size, int chunk, float scale, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (vdim <= 0 || vdim > kMaxValueDim) LLM_FAIL(-1, "talking attention: value size %d is not in [1, %d]", vdim, kMaxValueDim);
    if (kv_heads <= 0 || heads % kv_heads) LLM_FAIL(-1, "talking attention: heads %d is not a multiple of kv_heads %d", heads, kv_heads);
    if (heads > 64) LLM_FAIL(-1, "talking attention: %d heads (at most 64)", heads);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        const int per16 = 16 / (int)sizeof(T);        // elements of a 16-byte load
        const int vec = (dim % per16 == 0 && vdim % per16 == 0 && page_stride % per16 == 0) ? 1 : 0;
#define LLM_TALK(HPW)                                                                                                   \
    launch_talking<T, HPW>(q, q_stride, cache, page_stride, v_off, block_table, table_width, token_request, positions,  \
                           talk, slopes, out, out_stride, tokens, heads, kv_heads, dim, vdim, page_size, chunk, scale,  \
                           vec, stream)
        // Many tokens (prompt portions): at most eight warps a block, so that several blocks share an SM and hide each
        // other's loads.  Few tokens (decoded ones): a warp for every head or two, since the block's own width is all the
        // parallelism there is.  (2,048 tokens, 32 heads of 64: 468 -> 381 us; 8 tokens: 78 against 96 us the other way round.)
        const bool many = tokens >= 2 * 148;
        if (heads <= 8) return LLM_TALK(1);
        if (heads <= 16) return many ? LLM_TALK(2) : LLM_TALK(1);
        if (heads <= 32) return many ? LLM_TALK(4) : LLM_TALK(2);
        return many ? LLM_TALK(8) : LLM_TALK(4);
#undef LLM_TALK
    });
}

LLM_TRACE_EXPORT(talking_attention)
