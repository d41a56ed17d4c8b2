// Retention: linear attention with a fixed decay per head, as a scan over each request's tokens.
//     S_t = decay_h * S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t         S [dim, vdim] float32 per request and head
// q and k are rotated on their leading `2 * half` dims (pairs (i, i + half), angles from float32 cos/sin tables of
// the step's positions) and k is scaled, all in float32, by a kernel of its own ahead of the walk.
//
// The columns of S evolve independently (column c needs v_t[c] only), so a block owns `cpb` columns of one head of
// one request and walks the request's tokens in order; the `dim` rows of a column are shared out over `ds` neighbouring
// lanes (each keeps R of them in registers) whose partial outputs a shuffle adds.  The launcher picks R (and so the
// number of blocks, vdim / cpb per head and request) so that the grid fills the machine: the walk itself cannot be cut.
// The rows of the next block of tokens travel to shared memory (cp.async) while the current block is walked.
// Measured on B200 (2,048 tokens of one request, 32 heads): head sizes 64 / 64: 0.63 ms in segments, head sizes 128 / 128:
// 1.7 ms whole.  What bounds it is the count of instructions a token costs a warp (about a hundred for 24 useful
// multiply-adds at eight rows a thread: addresses from the run-time lane split, the shuffles of the sum), not memory.
// The walk is the same whatever the step's cut, so a portion continues bit for bit where the one before it stopped.
//
// A long portion is walked in two passes so that the walk is cut after all: pass one walks segments of `seg_len` tokens
// side by side, each from zero (a request's first from its state), and leaves what each gathered; pass two gives every
// later segment the state that stood at its start, S_in = sum over earlier segments of decay^(tokens in between) * gathered,
// adds decay^(n + 1) * S_in^T q to its n-th token, and the request's last segment leaves the state.  Where segments are
// cut depends on where the portion starts, which moves results by rounding only.
//
// The state is kept transposed, [slot, head, vdim, dim], so that the lanes that share a column read neighbouring words.
//
// `retention_headnorm_gate` then divides every head of o by its root mean square and multiplies by silu(gate).
#include "common.cuh"

namespace {

constexpr int kThreads = 128;
constexpr int kTargetBlocks = 2 * 148;
constexpr int kTokenBlock = 16;
constexpr int kSegment = 128;        // tokens of a segment, about (see the launcher)
constexpr int kMaxSegments = 32;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// q and k of every token and head, rotated and (k) scaled, as float32 [tokens, heads, 2, dim]: done once, ahead of the
// walk, so that the blocks that share a head's rows (one per `cpb` columns) do not each rotate them again.
template <typename T>
__global__ void __launch_bounds__(128)
retention_rotate_kernel(const T* __restrict__ proj, int proj_stride, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, int half, float* __restrict__ qk, int heads, int dim,
                        float k_scale, long long rows) {
    pdl_trigger();
    pdl_wait();
    const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);     // (token, head)
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const long long t = row / heads;
    const int h = (int)(row % heads);
    const T* q = proj + (size_t)t * proj_stride + (size_t)h * dim;
    const T* k = q + (size_t)heads * dim;
    float* dst = qk + (size_t)row * 2 * dim;
    const int rot = 2 * half;
    for (int d = lane; d < dim; d += 32) {
        float qv = to_f32(q[d]), kv = to_f32(k[d]);
        if (d < rot) {
            const bool first = d < half;
            const int i = first ? d : d - half, pd = first ? d + half : d - half;
            const float cs = cos_t[(size_t)t * half + i], sn = sin_t[(size_t)t * half + i];
            const float qp = to_f32(q[pd]), kp = to_f32(k[pd]);
            qv = first ? qv * cs - qp * sn : qv * cs + qp * sn;
            kv = first ? kv * cs - kp * sn : kv * cs + kp * sn;
        }
        dst[d] = qv;
        dst[dim + d] = kv * k_scale;
    }
}

// Rows [t0, t0 + nb) of the rotated q and k of head h (float32, `dim` each) and of this block's `cpb` value columns (as
// stored) into one stage: qs [tb, dim], ks [tb, dim] float32, then raw values [tb, cpb].
template <typename T>
__device__ __forceinline__ void stage_rows(float* qs, float* ks, T* rawv, const float* __restrict__ qk, const T* __restrict__ proj,
                                           int proj_stride, int heads, int h, int t0, int nb, int dim, int cpb, size_t v_col,
                                           int vcols, bool vec_qk, bool vec_v) {
    constexpr int kPer = 16 / (int)sizeof(T);
    if (vec_qk) {
        const int per_row = dim / 4;             // 16-byte pieces of a row; a token's q row and k row follow each other
        for (int idx = threadIdx.x; idx < nb * 2 * per_row; idx += blockDim.x) {
            const int tt = idx / (2 * per_row), x = idx % (2 * per_row);
            const float* src = qk + ((size_t)(t0 + tt) * heads + h) * 2 * dim + (size_t)x * 4;
            float* dst = x < per_row ? qs + tt * dim + x * 4 : ks + tt * dim + (x - per_row) * 4;
            cp_async16(dst, src);
        }
    } else {
        for (int idx = threadIdx.x; idx < nb * 2 * dim; idx += blockDim.x) {
            const int tt = idx / (2 * dim), x = idx % (2 * dim);
            const float v = qk[((size_t)(t0 + tt) * heads + h) * 2 * dim + x];
            if (x < dim) qs[tt * dim + x] = v;
            else ks[tt * dim + x - dim] = v;
        }
    }
    if (vec_v) {
        const int vper = cpb / kPer;
        for (int idx = threadIdx.x; idx < nb * vper; idx += blockDim.x) {
            const int tt = idx / vper, x = (idx % vper) * kPer;
            cp_async16(rawv + tt * cpb + x, proj + (size_t)(t0 + tt) * proj_stride + v_col + x);
        }
    } else {
        for (int idx = threadIdx.x; idx < nb * cpb; idx += blockDim.x) {
            const int tt = idx / cpb, x = idx % cpb;
            rawv[tt * cpb + x] = x < vcols ? proj[(size_t)(t0 + tt) * proj_stride + v_col + x] : from_f32<T>(0.f);
        }
    }
    cp_async_commit();
}

// MODE 0 walks; MODE 1 is the second pass of a walk that was cut into segments (see the launcher).
template <typename T, int R, int MODE>
__global__ void __launch_bounds__(kThreads)
retention_scan_kernel(const T* __restrict__ proj, int proj_stride, const float* __restrict__ qk,
                      const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ state_slots, const int* __restrict__ cu_seqlens,
                      float* __restrict__ out, int heads, int dim, int vdim, int ds, int cpb, int write, int vec,
                      int nseg, int seg_len, float* __restrict__ seg_state) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    constexpr int tb = kTokenBlock;
    // two stages of: q rows [tb, dim], k rows [tb, dim] (float32, as the rotation left them), value columns [tb, cpb] as stored
    const size_t stage_bytes = sizeof(float) * 2 * tb * dim + sizeof(T) * tb * cpb;
    float* vs = reinterpret_cast<float*>(smem_bytes + 2 * stage_bytes);        // [tb, cpb] float32
    const int h = blockIdx.y;
    // segment `seg` of request b: MODE 0 has a block for each, MODE 1 for all but a request's first
    const int b = MODE == 0 ? blockIdx.z / nseg : blockIdx.z / (nseg - 1);
    const int seg = MODE == 0 ? blockIdx.z % nseg : blockIdx.z % (nseg - 1) + 1;
    const int s = threadIdx.x % ds, cl = threadIdx.x / ds;
    const int c0 = blockIdx.x * cpb;
    const int c = c0 + cl;
    const bool live = c < vdim;
    const int vcols = min(cpb, vdim - c0);
    const bool vvec = vec && vcols == cpb;
    const int req_begin = cu_seqlens[b], req_end = cu_seqlens[b + 1];
    const int begin = nseg > 1 ? min(req_end, req_begin + seg * seg_len) : req_begin;
    const int end = nseg > 1 ? min(req_end, begin + seg_len) : req_end;
    if (begin >= end) return;                // the request is shorter than this segment's start (the whole block leaves)
    const float dec = decay[h];
    float* st = state + (((size_t)state_slots[b] * heads + h) * vdim + (live ? c : 0)) * dim;
    // where segment j of this (request, head, column) leaves what it gathered from zero (segment 0: from the state)
    float* sg = seg_state ? seg_state + ((((size_t)b * nseg) * heads + h) * vdim + (live ? c : 0)) * dim : nullptr;
    const size_t sg_stride = (size_t)heads * vdim * dim;
    float S[R];
    if (MODE == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = s + ds * r;
            S[r] = (live && d < dim && seg == 0) ? st[d] : 0.f;
        }
    } else {
        // the state at this segment's start: what the segments before it gathered, each decayed over those after it
        const float dl = powf(dec, (float)seg_len);
#pragma unroll
        for (int r = 0; r < R; ++r) S[r] = 0.f;
        for (int j = 0; j < seg; ++j) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int d = s + ds * r;
                if (live && d < dim) S[r] = fmaf(dl, S[r], sg[(size_t)j * sg_stride + d]);
            }
        }
    }
    const size_t v_col = 2 * (size_t)heads * dim + (size_t)h * vdim + c0;
    const bool vec_qk = dim % 4 == 0;
    auto stage_q = [&](int st_) { return reinterpret_cast<float*>(smem_bytes + st_ * stage_bytes); };
    auto stage_v = [&](int st_) { return reinterpret_cast<T*>(smem_bytes + st_ * stage_bytes + sizeof(float) * 2 * tb * dim); };
    stage_rows<T>(stage_q(0), stage_q(0) + tb * dim, stage_v(0), qk, proj, proj_stride, heads, h, begin, min(tb, end - begin), dim, cpb,
                  v_col, vcols, vec_qk, vvec);
    int stage = 0;
    float carried = 1.f;
    for (int t0 = begin; t0 < end; t0 += tb, stage ^= 1) {
        const int nb = min(tb, end - t0);
        const float* qs = stage_q(stage);
        const float* ks = qs + tb * dim;
        const T* rawv = stage_v(stage);
        cp_async_wait_all();
        __syncthreads();                     // the staged rows have landed; everybody is done with the other stage and with vs
        if (t0 + tb < end)                   // the next block's rows travel while this one is walked
            stage_rows<T>(stage_q(stage ^ 1), stage_q(stage ^ 1) + tb * dim, stage_v(stage ^ 1), qk, proj, proj_stride, heads, h, t0 + tb,
                          min(tb, end - t0 - tb), dim, cpb, v_col, vcols, vec_qk, vvec);
        for (int idx = threadIdx.x; idx < nb * cpb; idx += blockDim.x)
            vs[idx] = (idx % cpb) < vcols ? to_f32(rawv[idx]) : 0.f;
        __syncthreads();
        for (int tt = 0; tt < nb; ++tt) {
            const float* qr = qs + tt * dim;
            float part = 0.f;
            if (MODE == 0) {
                const float vv = vs[tt * cpb + cl];
                const float* kr = ks + tt * dim;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int d = s + ds * r;
                    if (d < dim) {
                        S[r] = fmaf(dec, S[r], kr[d] * vv);
                        part = fmaf(S[r], qr[d], part);
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const int d = s + ds * r;
                    if (d < dim) part = fmaf(S[r], qr[d], part);
                }
            }
            for (int o = ds >> 1; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            float* o_at = out + (size_t)(t0 + tt) * heads * vdim + (size_t)h * vdim + c;
            if (MODE == 0) {
                if (live && s == 0) *o_at = part;
            } else {
                carried *= dec;              // decay^(tokens of this segment up to and including this one)
                if (live && s == 0) *o_at += carried * part;
            }
        }
    }
    if (!live) return;
    if (MODE == 0) {
        if (nseg > 1) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int d = s + ds * r;
                if (d < dim) sg[(size_t)seg * sg_stride + d] = S[r];
            }
        }
        // a request of one segment is done after this pass
        if (write && seg == 0 && end == req_end) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int d = s + ds * r;
                if (d < dim) st[d] = S[r];
            }
        }
    } else if (write && end == req_end) {
        // the request's last segment leaves the state: what stood at its start, decayed over it, and what it gathered
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int d = s + ds * r;
            if (d < dim) st[d] = fmaf(carried, S[r], sg[(size_t)seg * sg_stride + d]);
        }
    }
}

// The same walk with a register tile: a thread keeps RG groups of four neighbouring rows of four neighbouring columns, so
// one 16-byte read of k, of q and of v feeds sixteen multiply-adds each (the plain form above reads a word per multiply-add
// and is what other sizes fall back to).  A column group's rows are shared out over `ds` lanes, rows 4 * (s + ds * g) ..+3 for
// lane s; the four column sums travel through a butterfly that halves what is sent at each of its first two steps.
// Needs dim and vdim to be multiples of 4.  (2,048 tokens, 32 heads of 128 / 128: 1.71 ms with the plain form.)
template <typename T, int RG, int MODE>
__global__ void __launch_bounds__(kThreads)
retention_tile_kernel(const T* __restrict__ proj, int proj_stride, const float* __restrict__ qk,
                      const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ state_slots,
                      const int* __restrict__ cu_seqlens, float* __restrict__ out, int heads, int dim, int vdim, int ds, int cpb,
                      int write, int vec, int nseg, int seg_len, float* __restrict__ seg_state) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_bytes[];
    constexpr int tb = kTokenBlock;
    const size_t stage_bytes = sizeof(float) * 2 * tb * dim + sizeof(T) * tb * cpb;
    float* vs = reinterpret_cast<float*>(smem_bytes + 2 * stage_bytes);        // [tb, cpb] float32
    const int h = blockIdx.y;
    const int b = MODE == 0 ? blockIdx.z / nseg : blockIdx.z / (nseg - 1);
    const int seg = MODE == 0 ? blockIdx.z % nseg : blockIdx.z % (nseg - 1) + 1;
    const int s = threadIdx.x % ds, cg = threadIdx.x / ds;
    const int c0 = blockIdx.x * cpb;
    const int c = c0 + 4 * cg;                       // the first of this thread's four columns
    const bool live = c < vdim;                      // (vdim is a multiple of 4: all four or none)
    const int vcols = min(cpb, vdim - c0);
    const bool vvec = vec && vcols == cpb;
    const int req_begin = cu_seqlens[b], req_end = cu_seqlens[b + 1];
    const int begin = nseg > 1 ? min(req_end, req_begin + seg * seg_len) : req_begin;
    const int end = nseg > 1 ? min(req_end, begin + seg_len) : req_end;
    if (begin >= end) return;
    const float dec = decay[h];
    float* st = state + (((size_t)state_slots[b] * heads + h) * vdim + (live ? c : 0)) * dim;
    float* sg = seg_state ? seg_state + ((((size_t)b * nseg) * heads + h) * vdim + (live ? c : 0)) * dim : nullptr;
    const size_t sg_stride = (size_t)heads * vdim * dim;
    float S[RG][4][4];                               // [row group][row][column]
    bool rows_live[RG];
#pragma unroll
    for (int g = 0; g < RG; ++g) rows_live[g] = live && 4 * (s + ds * g) < dim;
    auto load_state = [&](const float* src, float scale) {      // S = scale * S + src
#pragma unroll
        for (int g = 0; g < RG; ++g) {
            if (!rows_live[g]) continue;
            const int d = 4 * (s + ds * g);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 x = *reinterpret_cast<const float4*>(src + (size_t)j * dim + d);
                S[g][0][j] = fmaf(scale, S[g][0][j], x.x);
                S[g][1][j] = fmaf(scale, S[g][1][j], x.y);
                S[g][2][j] = fmaf(scale, S[g][2][j], x.z);
                S[g][3][j] = fmaf(scale, S[g][3][j], x.w);
            }
        }
    };
    auto store_state = [&](float* dst, const float* add, float scale) {   // dst = scale * S (+ add)
#pragma unroll
        for (int g = 0; g < RG; ++g) {
            if (!rows_live[g]) continue;
            const int d = 4 * (s + ds * g);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
                if (add) x = *reinterpret_cast<const float4*>(add + (size_t)j * dim + d);
                x.x = fmaf(scale, S[g][0][j], x.x);
                x.y = fmaf(scale, S[g][1][j], x.y);
                x.z = fmaf(scale, S[g][2][j], x.z);
                x.w = fmaf(scale, S[g][3][j], x.w);
                *reinterpret_cast<float4*>(dst + (size_t)j * dim + d) = x;
            }
        }
    };
#pragma unroll
    for (int g = 0; g < RG; ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) S[g][i][j] = 0.f;
    if (MODE == 0) {
        if (seg == 0) load_state(st, 0.f);
    } else {
        const float dl = powf(dec, (float)seg_len);
        for (int j = 0; j < seg; ++j) load_state(sg + (size_t)j * sg_stride, dl);
    }
    const size_t v_col = 2 * (size_t)heads * dim + (size_t)h * vdim + c0;
    auto stage_q = [&](int st_) { return reinterpret_cast<float*>(smem_bytes + st_ * stage_bytes); };
    auto stage_v = [&](int st_) { return reinterpret_cast<T*>(smem_bytes + st_ * stage_bytes + sizeof(float) * 2 * tb * dim); };
    stage_rows<T>(stage_q(0), stage_q(0) + tb * dim, stage_v(0), qk, proj, proj_stride, heads, h, begin, min(tb, end - begin), dim, cpb,
                  v_col, vcols, true, vvec);
    int stage = 0;
    float carried = 1.f;
    const int col_of_lane = ((s & 1) << 1) | ((s >> 1) & 1);      // whose sum this lane holds after the butterfly (ds >= 4)
    for (int t0 = begin; t0 < end; t0 += tb, stage ^= 1) {
        const int nb = min(tb, end - t0);
        const float* qs = stage_q(stage);
        const float* ks = qs + tb * dim;
        const T* rawv = stage_v(stage);
        cp_async_wait_all();
        __syncthreads();
        if (t0 + tb < end)
            stage_rows<T>(stage_q(stage ^ 1), stage_q(stage ^ 1) + tb * dim, stage_v(stage ^ 1), qk, proj, proj_stride, heads, h, t0 + tb,
                          min(tb, end - t0 - tb), dim, cpb, v_col, vcols, true, vvec);
        if (MODE == 0) {
            for (int idx = threadIdx.x; idx < nb * cpb; idx += blockDim.x)
                vs[idx] = (idx % cpb) < vcols ? to_f32(rawv[idx]) : 0.f;
            __syncthreads();
        }
        // second pass: what these tokens hold so far is asked for now and added to after the walk (four 16-byte pieces a thread
        // this way; a block wider than that takes the rest the slow way)
        float4 held[4];
        const int pieces = nb * (cpb >> 2);
        if (MODE == 1) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = threadIdx.x + u * kThreads;
                const int tt = idx / (cpb >> 2), x = (idx % (cpb >> 2)) << 2;
                if (idx < pieces && x < vcols)
                    held[u] = *reinterpret_cast<const float4*>(out + (size_t)(t0 + tt) * heads * vdim + (size_t)h * vdim + c0 + x);
            }
        }
        for (int tt = 0; tt < nb; ++tt) {
            float part[4] = {0.f, 0.f, 0.f, 0.f};
            float v4[4];
            if (MODE == 0) {
                const float4 x = *reinterpret_cast<const float4*>(vs + tt * cpb + 4 * cg);
                v4[0] = x.x; v4[1] = x.y; v4[2] = x.z; v4[3] = x.w;
            }
#pragma unroll
            for (int g = 0; g < RG; ++g) {
                if (!rows_live[g]) continue;
                const int d = 4 * (s + ds * g);
                const float4 qx = *reinterpret_cast<const float4*>(qs + tt * dim + d);
                const float q4[4] = {qx.x, qx.y, qx.z, qx.w};
                if (MODE == 0) {
                    const float4 kx = *reinterpret_cast<const float4*>(ks + tt * dim + d);
                    const float k4[4] = {kx.x, kx.y, kx.z, kx.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            S[g][i][j] = fmaf(dec, S[g][i][j], k4[i] * v4[j]);
                            part[j] = fmaf(S[g][i][j], q4[i], part[j]);
                        }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) part[j] = fmaf(S[g][i][j], q4[i], part[j]);
                }
            }
            if (MODE == 1) carried *= dec;
            float* o_at = out + (size_t)(t0 + tt) * heads * vdim + (size_t)h * vdim + c;
            if (ds >= 4) {
                const bool odd = s & 1, high = s & 2;
                const float r0 = __shfl_xor_sync(0xffffffffu, odd ? part[0] : part[2], 1);
                const float r1 = __shfl_xor_sync(0xffffffffu, odd ? part[1] : part[3], 1);
                const float a0 = (odd ? part[2] : part[0]) + r0, a1 = (odd ? part[3] : part[1]) + r1;
                float sum = (high ? a1 : a0) + __shfl_xor_sync(0xffffffffu, high ? a0 : a1, 2);
                for (int o = 4; o < ds; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (live && s < 4) {
                    if (MODE == 0) o_at[col_of_lane] = sum;
                    else vs[tt * cpb + 4 * cg + col_of_lane] = carried * sum;      // (the second pass has no use for values: vs collects what it adds)
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    for (int o = ds >> 1; o > 0; o >>= 1) part[j] += __shfl_xor_sync(0xffffffffu, part[j], o);
                if (live && s == 0) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (MODE == 0) o_at[j] = part[j];
                        else vs[tt * cpb + 4 * cg + j] = carried * part[j];
                    }
                }
            }
        }
        if (MODE == 1) {
            // what this block of tokens is to be given, added with all loads in flight at once
            __syncthreads();
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int idx = threadIdx.x + u * kThreads;
                const int tt = idx / (cpb >> 2), x = (idx % (cpb >> 2)) << 2;
                if (idx < pieces && x < vcols) {
                    const float4 add = *reinterpret_cast<const float4*>(vs + tt * cpb + x);
                    held[u].x += add.x; held[u].y += add.y; held[u].z += add.z; held[u].w += add.w;
                    *reinterpret_cast<float4*>(out + (size_t)(t0 + tt) * heads * vdim + (size_t)h * vdim + c0 + x) = held[u];
                }
            }
            for (int idx = threadIdx.x + 4 * kThreads; idx < pieces; idx += kThreads) {
                const int tt = idx / (cpb >> 2), x = (idx % (cpb >> 2)) << 2;
                if (x < vcols) {
                    float* o4 = out + (size_t)(t0 + tt) * heads * vdim + (size_t)h * vdim + c0 + x;
#pragma unroll
                    for (int e = 0; e < 4; ++e) o4[e] += vs[tt * cpb + x + e];
                }
            }
        }
    }
    if (!live) return;
    if (MODE == 0) {
        if (nseg > 1) store_state(sg + (size_t)seg * sg_stride, nullptr, 1.f);
        if (write && seg == 0 && end == req_end) store_state(st, nullptr, 1.f);
    } else if (write && end == req_end) {
        store_state(st, sg + (size_t)seg * sg_stride, carried);
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
// no rotation).  state [slots, heads, vdim, dim] float32 (transposed); out [tokens, heads * vdim] float32.
// `longest`: the most tokens one request brings; `seg_state`: scratch of `seg_state_floats` floats for the two-pass form
// (null: one pass); `qk_scratch`: tokens * heads * 2 * dim floats for the rotated q and k.  Returns the number of segments
// (1: one pass) or a negative code.  `target_blocks` (0: twice the SMs) and `segment_mode` move the launch rule for measurements.
LLM_API int llm_retention_scan(const void* proj, int proj_stride, const float* cos_t, const float* sin_t, int half,
                               const float* decay, float* state, const int* state_slots, const int* cu_seqlens,
                               float* out, int dtype, int tokens, int requests, int heads, int dim, int vdim, float k_scale,
                               int write, int longest, float* seg_state, long long seg_state_floats, float* qk_scratch,
                               int target_blocks, int segment_mode, cudaStream_t stream) {
    if (tokens == 0 || requests == 0) return 0;
    if (2 * half > dim) LLM_FAIL(-1, "retention: %d rotated dims exceed the head size %d", 2 * half, dim);
    if (dim > 1024) LLM_FAIL(-1, "retention: head size %d is too large (at most 1024)", dim);
    // segments: only where a request brings several hundred tokens and the walk as a whole has too few blocks for the machine
    // (two passes cost twice the arithmetic); as many as `seg_state` has room for
    int nseg = 1, seg_len = 0;
    const bool plain_only = segment_mode >= 4;          // (measurements: the form without a register tile)
    segment_mode &= 3;
    const bool tiled = dim % 4 == 0 && vdim % 4 == 0 && dim <= 4 * 32 * 4 && !plain_only;
    int min_ds = 1;
    while (min_ds * 4 < dim && min_ds < 32) min_ds *= 2;       // lanes per column (group) at the fewest rows a thread takes
    const int min_cpb = (tiled ? 4 : 1) * (kThreads / min_ds);
    const long long whole_blocks = (long long)requests * heads * ((vdim + min_cpb - 1) / min_cpb);
    if (target_blocks <= 0) target_blocks = kTargetBlocks;
    // segment_mode: 0 = by the rule above, 1 = never, 2 = wherever a request is long enough (measurements)
    if (longest >= 2 * kSegment && seg_state && segment_mode != 1 && (whole_blocks < target_blocks || segment_mode == 2)) {
        nseg = (longest + kSegment - 1) / kSegment;
        if (nseg > kMaxSegments) nseg = kMaxSegments;
        seg_len = ((longest + nseg - 1) / nseg + kTokenBlock - 1) / kTokenBlock * kTokenBlock;
        nseg = (longest + seg_len - 1) / seg_len;
        if ((long long)requests * nseg * heads * vdim * dim > seg_state_floats) nseg = 1;
    }
    int rows = 32, ds = 1, cpb = kThreads;
    if (tiled) {
        // row groups of four per thread: as many as still give the machine enough blocks
        for (rows = 4;; rows /= 2) {
            ds = 1;
            while (4 * ds * rows < dim) ds *= 2;
            if (ds <= 32) {
                cpb = 4 * (kThreads / ds);
                const long long blocks = (long long)requests * nseg * heads * ((vdim + cpb - 1) / cpb);
                // (a block wider than the head's columns would leave threads idle: fewer rows, more lanes per column then)
                if ((blocks >= target_blocks && cpb <= vdim) || rows == 1 || ds == 32) break;
            }
            if (rows == 1) break;
        }
    } else {
        // rows per thread: as many as still give the machine enough blocks (fewer rows = more lanes per column = more blocks)
        for (;; rows /= 2) {
            ds = 1;
            while (ds * rows < dim) ds *= 2;
            if (ds <= 32) {
                cpb = kThreads / ds;
                const long long blocks = (long long)requests * nseg * heads * ((vdim + cpb - 1) / cpb);
                if (blocks >= target_blocks || rows == 4 || ds == 32) break;
            }
            if (rows == 4) break;
        }
    }
    if (ds > 32) LLM_FAIL(-1, "retention: head size %d does not fit", dim);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        constexpr int kPer = 16 / (int)sizeof(T);
        const int vec = (dim % kPer == 0 && vdim % kPer == 0 && cpb % kPer == 0 && proj_stride % kPer == 0 &&
                         ((size_t)proj % 16) == 0) ? 1 : 0;                 // the value columns travel in 16-byte pieces
        const size_t smem = 2 * (sizeof(float) * 2 * kTokenBlock * dim + sizeof(T) * kTokenBlock * cpb) + sizeof(float) * kTokenBlock * cpb;
        const long long rows_qk = (long long)tokens * heads;
        llm_launch(retention_rotate_kernel<T>, (unsigned)((rows_qk + 3) / 4), 128, 0, stream, (const T*)proj, proj_stride, cos_t, sin_t,
                   half, qk_scratch, heads, dim, k_scale, rows_qk);
        LLM_CHECK_LAUNCH("retention_rotate");
        const unsigned gx = (vdim + cpb - 1) / cpb;
#define LLM_RET(KERNEL, RR, MODE, GZ)                                                                                      \
    do {                                                                                                                   \
        if (smem > 48 * 1024)                                                                                              \
            cudaFuncSetAttribute(KERNEL<T, RR, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
        llm_launch(KERNEL<T, RR, MODE>, dim3(gx, heads, GZ), kThreads, smem, stream, (const T*)proj, proj_stride,          \
                   (const float*)qk_scratch, decay, state, state_slots, cu_seqlens, out, heads, dim, vdim, ds, cpb, write,  \
                   vec, nseg, seg_len, nseg > 1 ? seg_state : (float*)nullptr);                                           \
    } while (0)
#define LLM_RET_ROWS(MODE, GZ)                                              \
    do {                                                                    \
        if (tiled) {                                                        \
            if (rows == 4) LLM_RET(retention_tile_kernel, 4, MODE, GZ);     \
            else if (rows == 2) LLM_RET(retention_tile_kernel, 2, MODE, GZ); \
            else LLM_RET(retention_tile_kernel, 1, MODE, GZ);               \
        } else if (rows == 32) LLM_RET(retention_scan_kernel, 32, MODE, GZ); \
        else if (rows == 16) LLM_RET(retention_scan_kernel, 16, MODE, GZ);  \
        else if (rows == 8) LLM_RET(retention_scan_kernel, 8, MODE, GZ);    \
        else LLM_RET(retention_scan_kernel, 4, MODE, GZ);                   \
    } while (0)
        LLM_RET_ROWS(0, requests * nseg);
        LLM_CHECK_LAUNCH("retention_scan");
        if (nseg > 1) {
            LLM_RET_ROWS(1, requests * (nseg - 1));
            LLM_CHECK_LAUNCH("retention_scan (second pass)");
        }
#undef LLM_RET_ROWS
#undef LLM_RET
        return nseg;
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
