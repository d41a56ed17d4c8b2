// Retention: linear attention with a fixed decay per head, as a scan over each request's tokens.
//     S_t = decay_h * S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t         S [dim, vdim] float32 per request and head
// q and k are rotated on their leading `2 * half` dims (pairs (i, i + half), angles from float32 cos/sin tables of
// the step's positions) and k is scaled, all in float32, as the rows are staged in shared memory.
//
// The columns of S evolve independently (column c needs v_t[c] only), so a block owns `cpb` columns of one head of
// one request and walks the request's tokens in order; the `dim` rows of a column are shared out over `ds` neighbouring
// lanes (each keeps up to kRows of them in registers) whose partial outputs a shuffle adds.  The walk is the same
// whatever the step's cut, so a portion continues bit for bit where the one before it stopped.
//
// `retention_headnorm_gate` then divides every head of o by its root mean square and multiplies by silu(gate).
#include "common.cuh"

namespace {

constexpr int kRows = 32;

template <typename T>
__global__ void __launch_bounds__(128)
retention_scan_kernel(const T* __restrict__ proj, int proj_stride, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int half, const float* __restrict__ decay,
                      float* __restrict__ state, const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens,
                      float* __restrict__ out, int heads, int dim, int vdim, int ds, int cpb, int tb, float k_scale,
                      int write) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float smem[];
    float* qs = smem;                    // [tb, dim]
    float* ks = qs + tb * dim;           // [tb, dim]
    float* vs = ks + tb * dim;           // [tb, cpb]
    const int h = blockIdx.y, b = blockIdx.z;
    const int s = threadIdx.x % ds, cl = threadIdx.x / ds;
    const int c = blockIdx.x * cpb + cl;
    const bool live = cl < cpb && c < vdim;
    const int begin = cu_seqlens[b], end = cu_seqlens[b + 1];
    const float dec = decay[h];
    float* st = state + ((size_t)state_slots[b] * heads + h) * dim * vdim;
    float S[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const int d = s + ds * r;
        S[r] = (live && d < dim) ? st[(size_t)d * vdim + c] : 0.f;
    }
    const int rot = 2 * half;
    const size_t q_col = (size_t)h * dim, k_col = (size_t)heads * dim + (size_t)h * dim;
    const size_t v_col = 2 * (size_t)heads * dim + (size_t)h * vdim;
    for (int t0 = begin; t0 < end; t0 += tb) {
        const int nb = min(tb, end - t0);
        for (int idx = threadIdx.x; idx < nb * dim; idx += blockDim.x) {
            const int tt = idx / dim, d = idx % dim;
            const T* row = proj + (size_t)(t0 + tt) * proj_stride;
            float qv = to_f32(row[q_col + d]), kv = to_f32(row[k_col + d]);
            if (d < rot) {
                const bool first = d < half;
                const int i = first ? d : d - half, pd = first ? d + half : d - half;
                const float cs = cos_t[(size_t)(t0 + tt) * half + i], sn = sin_t[(size_t)(t0 + tt) * half + i];
                const float qp = to_f32(row[q_col + pd]), kp = to_f32(row[k_col + pd]);
                qv = first ? qv * cs - qp * sn : qv * cs + qp * sn;
                kv = first ? kv * cs - kp * sn : kv * cs + kp * sn;
            }
            qs[idx] = qv;
            ks[idx] = kv * k_scale;
        }
        for (int idx = threadIdx.x; idx < nb * cpb; idx += blockDim.x) {
            const int tt = idx / cpb, cc = blockIdx.x * cpb + idx % cpb;
            vs[idx] = cc < vdim ? to_f32(proj[(size_t)(t0 + tt) * proj_stride + v_col + cc]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nb; ++tt) {
            const float vv = cl < cpb ? vs[tt * cpb + cl] : 0.f;
            const float* kr = ks + tt * dim;
            const float* qr = qs + tt * dim;
            float part = 0.f;
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const int d = s + ds * r;
                if (d < dim) {
                    S[r] = fmaf(dec, S[r], kr[d] * vv);
                    part = fmaf(S[r], qr[d], part);
                }
            }
            for (int o = ds >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (live && s == 0) out[(size_t)(t0 + tt) * heads * vdim + (size_t)h * vdim + c] = part;
        }
        __syncthreads();
    }
    if (write && live) {
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int d = s + ds * r;
            if (d < dim) st[(size_t)d * vdim + c] = S[r];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
headnorm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride, T* __restrict__ out,
                     long long items, int heads, int vdim, float eps) {
    pdl_trigger();
    pdl_wait();
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= items) return;
    const long long t = item / heads;
    const int h = (int)(item % heads);
    const float* x = o + (size_t)t * heads * vdim + (size_t)h * vdim;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) ss += x[d] * x[d];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    const T* g = gate + (size_t)t * gate_stride + (size_t)h * vdim;
    T* y = out + (size_t)t * heads * vdim + (size_t)h * vdim;
    for (int d = lane; d < vdim; d += 32) {
        const float z = to_f32(g[d]);
        y[d] = from_f32<T>(x[d] * inv * (z / (1.0f + expf(-z))));
    }
}

}  // namespace

// proj [tokens, proj_stride]: q of all heads, then k, then v (heads * vdim).  cos_t / sin_t [tokens, half] float32 (half = 0:
// no rotation).  state [slots, heads, dim, vdim] float32; out [tokens, heads * vdim] float32.
LLM_API int llm_retention_scan(const void* proj, int proj_stride, const float* cos_t, const float* sin_t, int half,
                               const float* decay, float* state, const int* state_slots, const int* cu_seqlens,
                               float* out, int dtype, int tokens, int requests, int heads, int dim, int vdim, float k_scale,
                               int write, cudaStream_t stream) {
    if (tokens == 0 || requests == 0) return 0;
    int ds = 1;
    while ((dim + ds - 1) / ds > kRows) ds *= 2;
    if (ds > 32) LLM_FAIL(-1, "retention: head size %d is too large (at most %d)", dim, 32 * kRows);
    if (2 * half > dim) LLM_FAIL(-1, "retention: %d rotated dims exceed the head size %d", 2 * half, dim);
    const int unit = 32 / ds;                                   // columns of one warp
    int cpb = 128 / ds;
    const int need = (vdim + unit - 1) / unit * unit;           // whole warps
    if (need < cpb) cpb = need;
    const int tb = dim <= 256 ? 16 : (dim <= 512 ? 8 : 4);
    const size_t smem = sizeof(float) * ((size_t)2 * tb * dim + (size_t)tb * cpb);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(retention_scan_kernel<T>, dim3((vdim + cpb - 1) / cpb, heads, requests), cpb * ds, smem, stream,
                   (const T*)proj, proj_stride, cos_t, sin_t, half, decay, state, state_slots, cu_seqlens, out, heads, dim,
                   vdim, ds, cpb, tb, k_scale, write);
        LLM_CHECK_LAUNCH("retention_scan");
        return 0;
    });
}

// out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * silu(gate[t, h, :]);  gate rows are `gate_stride` elements apart.
LLM_API int llm_retention_headnorm_gate(const float* o, const void* gate, int gate_stride, void* out, int dtype,
                                        int tokens, int heads, int vdim, float eps, cudaStream_t stream) {
    if (tokens == 0) return 0;
    const long long items = (long long)tokens * heads;
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(headnorm_gate_kernel<T>, (unsigned)((items + 3) / 4), 128, 0, stream, o, (const T*)gate, gate_stride,
                   (T*)out, items, heads, vdim, eps);
        LLM_CHECK_LAUNCH("retention_headnorm_gate");
        return 0;
    });
}

LLM_TRACE_EXPORT(retention)
