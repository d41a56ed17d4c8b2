// Talking-heads attention for prompt portions in bfloat16, on the tensor core (mma.sync m16n8k16), for chunked masks
// of up to 128 positions and up to 32 heads: a block takes a tile of up to 16 neighbouring query tokens of one request
// and all heads, because every head's score of a key enters every head's softmax.
//
//   1. per key/value head (two at a time, four warps each): the keys the tile can see (its first token's chunk start up to its last token: at most
//      chunk + 15) travel to shared memory once; a warp per query head computes S = Q K^T for the 16 x keys tile and
//      leaves scale * S - slope * distance in shared memory as float32, for all heads;
//   2. the mixing a[h] = sum_g talk[h, g] * s[g] in float32, a thread per (query, key), g ascending (the order of the
//      one-token kernel), in place; what a query may not see becomes -inf;
//   3. per key/value head (again two at a time): its values travel to shared memory transposed; a warp per query head runs the softmax of
//      its 16 rows in the layout of the product's left operand, rounds P to bfloat16 for P V only, and writes the rows out.
//
// The one-token kernel (talking_attention.cu) serves decoded tokens, float32, larger chunks and more heads.
#include "common.cuh"

namespace {

constexpr int kQ = 16;
constexpr int kWarps = 8;
constexpr int kSlots = 2;           // key/value heads in shared memory at a time; kWarps / kSlots warps work on each
constexpr int kMaxHeads = 32;
constexpr int kMaxDimSteps = 8;      // head size up to 128
constexpr int kMaxKeySteps = 9;      // up to 144 keys a tile

__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__global__ void __launch_bounds__(kWarps * 32)
talking_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, const __nv_bfloat16* __restrict__ cache,
                        long long page_stride, long long v_off, const int* __restrict__ block_table, int table_width,
                        const int* __restrict__ tiles, const float* __restrict__ talk, const float* __restrict__ slopes,
                        __nv_bfloat16* __restrict__ out, int out_stride, int heads, int kv_heads, int dim, int vdim,
                        int page_size, int chunk, float scale, int nkp) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int hp = (heads + 7) & ~7;
    float* S = reinterpret_cast<float*>(smem_raw);              // [heads, kQ, nkp]
    float* talk_s = S + (size_t)heads * kQ * nkp;               // [heads (g), hp (h)]
    float* slope_s = talk_s + heads * hp;                       // [heads] (padded to 8)
    __nv_bfloat16* tile_s = reinterpret_cast<__nv_bfloat16*>(slope_s + hp);   // keys [nkp, dim + 8], later values^T [vdim, nkp + 8]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int gq = lane >> 2, tq = lane & 3;                    // the fragment's row (and row + 8) and column pair
    const int4 tile = reinterpret_cast<const int4*>(tiles)[blockIdx.x];
    const int row0 = tile.x, nrows = tile.y, pos0 = tile.z;
    const int* table = block_table + (size_t)tile.w * table_width;
    const int lo = (pos0 / chunk) * chunk;
    const int nk = pos0 + nrows - lo;                           // keys lo .. pos0 + nrows - 1
    const int group = heads / kv_heads;
    const int kstride = dim + 8, vstride = nkp + 8;
    const int dsteps = dim >> 4, ksteps = nkp >> 4;
    const int slot_elems = max(nkp * kstride, vdim * vstride);
    constexpr int kWarpsPerSlot = kWarps / kSlots;
    const int slot = warp / kWarpsPerSlot, warp_in_slot = warp % kWarpsPerSlot;

    for (int i = threadIdx.x; i < heads * hp; i += blockDim.x) {
        const int g = i / hp, h = i % hp;
        talk_s[i] = h < heads ? talk[h * heads + g] : 0.f;
    }
    for (int i = threadIdx.x; i < hp; i += blockDim.x) slope_s[i] = i < heads ? slopes[i] : 0.f;

    // ---- 1. scores of every head ---------------------------------------------------------------------------
    for (int kv0 = 0; kv0 < kv_heads; kv0 += kSlots) {
        const int per_row = dim >> 3;                           // 16-byte pieces of a key row
        for (int idx = threadIdx.x; idx < kSlots * nkp * per_row; idx += blockDim.x) {
            const int sl = idx / (nkp * per_row), rem = idx % (nkp * per_row);
            const int n = rem / per_row, x = (rem % per_row) << 3;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (n < nk && kv0 + sl < kv_heads) {
                const int j = lo + n;
                const __nv_bfloat16* src = cache + (size_t)table[j / page_size] * page_stride +
                                           ((size_t)(kv0 + sl) * page_size + j % page_size) * dim + x;
                v = *reinterpret_cast<const uint4*>(src);
            }
            *reinterpret_cast<uint4*>(tile_s + sl * slot_elems + n * kstride + x) = v;
        }
        __syncthreads();
        const int kvh = kv0 + slot;
        for (int r = warp_in_slot; r < group && kvh < kv_heads; r += kWarpsPerSlot) {
            const int g = kvh * group + r;
            uint32_t a[kMaxDimSteps][4];
            const __nv_bfloat16* qa = q + (size_t)(row0 + gq) * q_stride + (size_t)g * dim + 2 * tq;
            const __nv_bfloat16* qb = qa + (size_t)8 * q_stride;
            const bool has_a = gq < nrows, has_b = gq + 8 < nrows;
#pragma unroll
            for (int ks = 0; ks < kMaxDimSteps; ++ks) {
                if (ks < dsteps) {
                    a[ks][0] = has_a ? *reinterpret_cast<const uint32_t*>(qa + ks * 16) : 0u;
                    a[ks][1] = has_b ? *reinterpret_cast<const uint32_t*>(qb + ks * 16) : 0u;
                    a[ks][2] = has_a ? *reinterpret_cast<const uint32_t*>(qa + ks * 16 + 8) : 0u;
                    a[ks][3] = has_b ? *reinterpret_cast<const uint32_t*>(qb + ks * 16 + 8) : 0u;
                }
            }
            const float slope = slope_s[g];
            float* Sg = S + (size_t)g * kQ * nkp;
            for (int nt = 0; nt < (nkp >> 3); ++nt) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                const __nv_bfloat16* kb = tile_s + slot * slot_elems + (nt * 8 + gq) * kstride + 2 * tq;
#pragma unroll
                for (int ks = 0; ks < kMaxDimSteps; ++ks) {
                    if (ks < dsteps)
                        mma_16816(c, a[ks], *reinterpret_cast<const uint32_t*>(kb + ks * 16),
                                  *reinterpret_cast<const uint32_t*>(kb + ks * 16 + 8));
                }
                const int n = nt * 8 + 2 * tq;
                const float da = (float)(pos0 + gq - (lo + n)), db = da + 8.f;      // distance of row gq (gq + 8) to key n
                *reinterpret_cast<float2*>(Sg + gq * nkp + n) = make_float2(scale * c[0] - slope * da, scale * c[1] - slope * (da - 1.f));
                *reinterpret_cast<float2*>(Sg + (gq + 8) * nkp + n) = make_float2(scale * c[2] - slope * db, scale * c[3] - slope * (db - 1.f));
            }
        }
        __syncthreads();
    }

    // ---- 2. the heads talk -----------------------------------------------------------------------------------
    for (int idx = threadIdx.x; idx < kQ * nkp; idx += blockDim.x) {
        const int i = idx / nkp, n = idx % nkp;
        const int pi = pos0 + i, j = lo + n;
        const bool visible = i < nrows && n < nk && j <= pi && j / chunk == pi / chunk;
        float acc[kMaxHeads];
#pragma unroll
        for (int h = 0; h < kMaxHeads; ++h) acc[h] = 0.f;
        for (int g = 0; g < heads; ++g) {
            const float sg = S[(size_t)g * kQ * nkp + idx];
            const float* trow = talk_s + g * hp;
#pragma unroll
            for (int h = 0; h < kMaxHeads; h += 4) {
                if (h < hp) {
                    const float4 w = *reinterpret_cast<const float4*>(trow + h);
                    acc[h] = fmaf(w.x, sg, acc[h]);
                    acc[h + 1] = fmaf(w.y, sg, acc[h + 1]);
                    acc[h + 2] = fmaf(w.z, sg, acc[h + 2]);
                    acc[h + 3] = fmaf(w.w, sg, acc[h + 3]);
                }
            }
        }
#pragma unroll
        for (int h = 0; h < kMaxHeads; ++h)
            if (h < heads) S[(size_t)h * kQ * nkp + idx] = visible ? acc[h] : -INFINITY;
    }
    __syncthreads();

    // ---- 3. softmax and P V -------------------------------------------------------------------------------
    for (int kv0 = 0; kv0 < kv_heads; kv0 += kSlots) {
        const int per_row = vdim >> 3;
        for (int idx = threadIdx.x; idx < kSlots * nkp * per_row; idx += blockDim.x) {
            const int sl = idx / (nkp * per_row), rem = idx % (nkp * per_row);
            const int n = rem / per_row, x = (rem % per_row) << 3;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (n < nk && kv0 + sl < kv_heads) {
                const int j = lo + n;
                const __nv_bfloat16* src = cache + (size_t)table[j / page_size] * page_stride + v_off +
                                           ((size_t)(kv0 + sl) * page_size + j % page_size) * vdim + x;
                v = *reinterpret_cast<const uint4*>(src);
            }
            const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
            for (int u = 0; u < 8; ++u) tile_s[sl * slot_elems + (x + u) * vstride + n] = e[u];
        }
        __syncthreads();
        const int kvh = kv0 + slot;
        for (int r = warp_in_slot; r < group && kvh < kv_heads; r += kWarpsPerSlot) {
            const int h = kvh * group + r;
            const float* Sa = S + (size_t)h * kQ * nkp + gq * nkp + 2 * tq;
            const float* Sb = Sa + 8 * nkp;
            float ma = -INFINITY, mb = -INFINITY;
#pragma unroll
            for (int ks = 0; ks < kMaxKeySteps; ++ks) {
                if (ks < ksteps) {
                    const float2 a0 = *reinterpret_cast<const float2*>(Sa + ks * 16), a1 = *reinterpret_cast<const float2*>(Sa + ks * 16 + 8);
                    const float2 b0 = *reinterpret_cast<const float2*>(Sb + ks * 16), b1 = *reinterpret_cast<const float2*>(Sb + ks * 16 + 8);
                    ma = fmaxf(ma, fmaxf(fmaxf(a0.x, a0.y), fmaxf(a1.x, a1.y)));
                    mb = fmaxf(mb, fmaxf(fmaxf(b0.x, b0.y), fmaxf(b1.x, b1.y)));
                }
            }
            ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 1));
            ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, 2));
            mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 1));
            mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, 2));
            if (ma == -INFINITY) ma = 0.f;        // a row past the tile's last token: all weights 0, nothing written
            if (mb == -INFINITY) mb = 0.f;
            uint32_t p[kMaxKeySteps][4];
            float la = 0.f, lb = 0.f;
#pragma unroll
            for (int ks = 0; ks < kMaxKeySteps; ++ks) {
                if (ks < ksteps) {
                    const float2 a0 = *reinterpret_cast<const float2*>(Sa + ks * 16), a1 = *reinterpret_cast<const float2*>(Sa + ks * 16 + 8);
                    const float2 b0 = *reinterpret_cast<const float2*>(Sb + ks * 16), b1 = *reinterpret_cast<const float2*>(Sb + ks * 16 + 8);
                    const float pa0 = expf(a0.x - ma), pa1 = expf(a0.y - ma), pa2 = expf(a1.x - ma), pa3 = expf(a1.y - ma);
                    const float pb0 = expf(b0.x - mb), pb1 = expf(b0.y - mb), pb2 = expf(b1.x - mb), pb3 = expf(b1.y - mb);
                    la += (pa0 + pa1) + (pa2 + pa3);
                    lb += (pb0 + pb1) + (pb2 + pb3);
                    p[ks][0] = pack_bf16(pa0, pa1);
                    p[ks][1] = pack_bf16(pb0, pb1);
                    p[ks][2] = pack_bf16(pa2, pa3);
                    p[ks][3] = pack_bf16(pb2, pb3);
                }
            }
            la += __shfl_xor_sync(0xffffffffu, la, 1);
            la += __shfl_xor_sync(0xffffffffu, la, 2);
            lb += __shfl_xor_sync(0xffffffffu, lb, 1);
            lb += __shfl_xor_sync(0xffffffffu, lb, 2);
            const float ia = la > 0.f ? 1.0f / la : 0.f, ib = lb > 0.f ? 1.0f / lb : 0.f;
            __nv_bfloat16* oa = out + (size_t)(row0 + gq) * out_stride + (size_t)h * vdim + 2 * tq;
            __nv_bfloat16* ob = oa + (size_t)8 * out_stride;
            for (int nt = 0; nt < (vdim >> 3); ++nt) {
                float c[4] = {0.f, 0.f, 0.f, 0.f};
                const __nv_bfloat16* vb = tile_s + slot * slot_elems + (nt * 8 + gq) * vstride + 2 * tq;
#pragma unroll
                for (int ks = 0; ks < kMaxKeySteps; ++ks) {
                    if (ks < ksteps)
                        mma_16816(c, p[ks], *reinterpret_cast<const uint32_t*>(vb + ks * 16),
                                  *reinterpret_cast<const uint32_t*>(vb + ks * 16 + 8));
                }
                if (gq < nrows) *reinterpret_cast<__nv_bfloat162*>(oa + nt * 8) = __floats2bfloat162_rn(c[0] * ia, c[1] * ia);
                if (gq + 8 < nrows) *reinterpret_cast<__nv_bfloat162*>(ob + nt * 8) = __floats2bfloat162_rn(c[2] * ib, c[3] * ib);
            }
        }
        __syncthreads();
    }
}

size_t mma_smem_bytes(int heads, int dim, int vdim, int nkp) {
    const int hp = (heads + 7) & ~7;
    const size_t tile = sizeof(__nv_bfloat16) * (size_t)((nkp * (dim + 8)) > (vdim * (nkp + 8)) ? nkp * (dim + 8) : vdim * (nkp + 8));
    return sizeof(float) * ((size_t)heads * kQ * nkp + (size_t)heads * hp + hp) + kSlots * tile;
}

int keys_padded(int chunk) { return (chunk + kQ - 1 + 15) / 16 * 16; }

}  // namespace

// 1 if the tensor-core form takes these sizes (bfloat16 only): a chunked mask of 1 to 128 positions, at most 32 heads,
// key heads of a multiple of 16 up to 128, value heads of a multiple of 8, and a tile's scores that fit shared memory.
LLM_API int llm_talking_attention_mma_supported(int heads, int kv_heads, int dim, int vdim, int chunk, long long page_stride) {
    if (chunk <= 0 || chunk > 128 || heads > kMaxHeads || kv_heads <= 0 || heads % kv_heads) return 0;
    if (dim % 16 || dim > 16 * kMaxDimSteps || vdim % 8 || vdim <= 0 || page_stride % 8) return 0;
    const int nkp = keys_padded(chunk);
    if (nkp > 16 * kMaxKeySteps) return 0;
    return mma_smem_bytes(heads, dim, vdim, nkp) <= 224 * 1024 ? 1 : 0;
}

// tiles [n_tiles, 4] int32: first token row, rows (1 to 16), position of the first row, request (row of the block table).
LLM_API int llm_talking_attention_mma(const void* q, int q_stride, const void* cache, long long page_stride, long long v_off,
                                      const int* block_table, int table_width, const int* tiles, int n_tiles,
                                      const float* talk, const float* slopes, void* out, int out_stride, int heads,
                                      int kv_heads, int dim, int vdim, int page_size, int chunk, float scale,
                                      cudaStream_t stream) {
    if (n_tiles == 0) return 0;
    if (!llm_talking_attention_mma_supported(heads, kv_heads, dim, vdim, chunk, page_stride))
        LLM_FAIL(-1, "talking attention (tensor core): sizes not supported (heads %d, dim %d, vdim %d, chunk %d)", heads, dim, vdim, chunk);
    if (q_stride % 2 || out_stride % 2) LLM_FAIL(-1, "talking attention (tensor core): odd row strides");
    const int nkp = keys_padded(chunk);
    const size_t smem = mma_smem_bytes(heads, dim, vdim, nkp);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(talking_attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    llm_launch(talking_attn_mma_kernel, n_tiles, kWarps * 32, smem, stream, (const __nv_bfloat16*)q, q_stride,
               (const __nv_bfloat16*)cache, page_stride, v_off, block_table, table_width, tiles, talk, slopes,
               (__nv_bfloat16*)out, out_stride, heads, kv_heads, dim, vdim, page_size, chunk, scale, nkp);
    LLM_CHECK_LAUNCH("talking_attention_mma");
    return 0;
}

LLM_TRACE_EXPORT(talking_attention_mma)
