"""Plain-torch restatements of every kernel of the engine's kernel set, one function per
kernel, float32 arithmetic.  Two uses:
  * the `-m gpu` tests compare each CUDA kernel alone with its function here;
  * the CPU tests hand a `TorchKernels` object to the engine in place of the CUDA kernel
    set, which exercises the host logic (cache manager, step function, scheduler, replay)
    on a box without a GPU.  The engine itself has no such path.
"""
import math

import numpy as np
import torch


def ref_embed(ids, table, scale=1.0):
    return table[ids.long()].float() * scale


def ref_add_rmsnorm(residual, delta, weight, eps, rows=None, out_dtype=torch.float32):
    """Returns (new residual, normed)."""
    v = residual.float() + (delta.float() if delta is not None else 0)
    src = v if rows is None else v[rows.long()]
    y = src * torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return v, y.to(out_dtype)


def ref_rope(qkv, positions, inv_freq, heads, kv_heads, head_dim, rotary_dim):
    """Rotates the query and key heads of qkv rows; returns a new [T, (H+2Hkv)*D] float tensor."""
    T = qkv.shape[0]
    x = qkv.float().view(T, heads + 2 * kv_heads, head_dim).clone()
    if rotary_dim:
        ang = positions.float().unsqueeze(1) * inv_freq.float().unsqueeze(0)      # [T, rot/2]
        c, s = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
        half = rotary_dim // 2
        rot = x[:, :heads + kv_heads]
        x1, x2 = rot[..., :half].clone(), rot[..., half:rotary_dim].clone()
        rot[..., :half] = x1 * c - x2 * s
        rot[..., half:rotary_dim] = x2 * c + x1 * s
    return x.view(T, -1)


def ref_store(cache_layer, rotated, slots, heads, kv_heads, head_dim):
    """cache_layer [pages, 2, Hkv, page, D]; writes k and v rows of `rotated` at `slots`."""
    T = rotated.shape[0]
    page_size = cache_layer.shape[3]
    x = rotated.view(T, heads + 2 * kv_heads, head_dim)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        p, o = divmod(s, page_size)
        cache_layer[p, 0, :, o, :] = x[t, heads:heads + kv_heads].to(cache_layer.dtype)
        cache_layer[p, 1, :, o, :] = x[t, heads + kv_heads:].to(cache_layer.dtype)


def ref_paged_attention(q, cache_layer, block_table, token_request, positions, heads, kv_heads, head_dim,
                        window=0, scale=0.0):
    """q [T, >= heads*head_dim] (query heads first); returns [T, heads*head_dim] float32."""
    T = q.shape[0]
    page_size = cache_layer.shape[3]
    scale = scale or 1.0 / math.sqrt(head_dim)
    group = heads // kv_heads
    out = torch.zeros(T, heads, head_dim, dtype=torch.float32, device=q.device)
    for t in range(T):
        pos = int(positions[t])
        lo = max(0, pos - window + 1) if window > 0 else 0
        table = block_table[int(token_request[t])]
        idx = torch.arange(lo, pos + 1, device=q.device)
        pages = table[(idx // page_size).long()].long()
        offs = (idx % page_size).long()
        k = cache_layer[pages, 0, :, offs, :].float()        # [n, Hkv, D]
        v = cache_layer[pages, 1, :, offs, :].float()
        qt = q[t, :heads * head_dim].float().view(heads, head_dim)
        kk = k.repeat_interleave(group, dim=1)                # [n, H, D]
        vv = v.repeat_interleave(group, dim=1)
        sc = torch.einsum("hd,nhd->hn", qt, kk) * scale
        p = torch.softmax(sc, dim=-1)
        out[t] = torch.einsum("hn,nhd->hd", p, vv)
    return out.view(T, heads * head_dim)


def ref_linear(x, weight, swiglu=False):
    y = x.float() @ weight.float().t()
    if swiglu:
        n = weight.shape[0] // 2
        return torch.nn.functional.silu(y[:, :n]) * y[:, n:]
    return y


def ref_silu_mul(gu):
    n = gu.shape[1] // 2
    g = gu.float()
    return torch.nn.functional.silu(g[:, :n]) * g[:, n:]



def ref_conv_norm_store(u, bias, taps_w, q_gain, k_gain, state, state_slots, cu_seqlens, heads, kv_heads, head_dim,
                        value_dim, eps, own_kv):
    """The short convolution with its norms.  u [T, C]; state [slots, taps - 1, C] float32 or None (one tap).
    Returns (q [T, H*D], k [T, G*D] | None, v [T, G*V] | None, new state rows {slot: [taps - 1, C]})."""
    T, C = u.shape
    n = taps_w.shape[1] if taps_w is not None else 1
    x = u.float() + (bias.float() if bias is not None else 0)
    y = torch.zeros_like(x)
    new_state = {}
    cu = [int(c) for c in cu_seqlens]
    for b in range(len(cu) - 1):
        lo, hi = cu[b], cu[b + 1]
        slot = int(state_slots[b])
        if taps_w is not None:
            full = torch.cat([state[slot].float(), x[lo:hi]]) if n > 1 else x[lo:hi]          # [n - 1 + rows, C]
            y[lo:hi] = sum(taps_w[:, j].float() * full[j:j + hi - lo] for j in range(n))
            if n > 1:
                new_state[slot] = full[-(n - 1):].clone()
        else:
            y[lo:hi] = x[lo:hi]
    cq = heads * head_dim
    def rms(z):
        return z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + eps)
    q = rms(y[:, :cq]) * q_gain.float()
    if not own_kv:
        return q, None, None, new_state
    ck = kv_heads * head_dim
    k = rms(y[:, cq:cq + ck]) * k_gain.float()
    v = rms(y[:, cq + ck:].view(T, kv_heads, value_dim)).reshape(T, kv_heads * value_dim)
    return q, k, v, new_state


def ref_talking_attention(q, cache, block_table, token_request, positions, talk, slopes, heads, kv_heads, head_dim,
                          value_dim, page_size, chunk, scale):
    """q [T, H*D]; cache [pages, kv_heads*page*(D+V)] (key plane, then value plane); returns [T, H*V] float32."""
    T = q.shape[0]
    group = heads // kv_heads
    kplane = cache[:, :kv_heads * page_size * head_dim].view(-1, kv_heads, page_size, head_dim)
    vplane = cache[:, kv_heads * page_size * head_dim:].view(-1, kv_heads, page_size, value_dim)
    out = torch.zeros(T, heads, value_dim, dtype=torch.float32, device=q.device)
    for t in range(T):
        pos = int(positions[t])
        lo = (pos // chunk) * chunk if chunk > 0 else 0
        idx = torch.arange(lo, pos + 1, device=q.device)
        table = block_table[int(token_request[t])]
        pages, offs = table[(idx // page_size).long()].long(), (idx % page_size).long()
        k = kplane[pages, :, offs, :].float().repeat_interleave(group, dim=1)        # [n, H, D]
        v = vplane[pages, :, offs, :].float().repeat_interleave(group, dim=1)        # [n, H, V]
        qt = q[t].float().view(heads, head_dim)
        s = torch.einsum("hd,nhd->hn", qt, k) * scale - slopes.float().view(heads, 1) * (pos - idx).float().view(1, -1)
        a = talk.float() @ s
        out[t] = torch.einsum("hn,nhv->hv", torch.softmax(a, dim=-1), v)
    return out.view(T, heads * value_dim)


def ref_retention(proj, cos, sin, rotary_dim, decay, state, state_slots, cu_seqlens, heads, head_dim, value_dim, k_scale):
    """proj [T, q | k | v | ...]; state [slots, H, V, D] float32, S transposed (read, and returned updated as {slot: [H, V, D]});
    returns (o [T, H*V] float32, new states)."""
    T = proj.shape[0]
    qk = heads * head_dim
    q = proj[:, :qk].float().view(T, heads, head_dim).clone()
    k = proj[:, qk:2 * qk].float().view(T, heads, head_dim).clone()
    v = proj[:, 2 * qk:2 * qk + heads * value_dim].float().view(T, heads, value_dim)
    if rotary_dim:
        half = rotary_dim // 2
        c, s = cos.float().view(T, 1, half), sin.float().view(T, 1, half)
        for x in (q, k):
            a, b = x[..., :half].clone(), x[..., half:rotary_dim].clone()
            x[..., :half] = a * c - b * s
            x[..., half:rotary_dim] = b * c + a * s
    k = k * k_scale
    o = torch.zeros(T, heads, value_dim, dtype=torch.float32, device=proj.device)
    new = {}
    cu = [int(c) for c in cu_seqlens]
    d = decay.float().view(heads, 1, 1)
    for b in range(len(cu) - 1):
        slot = int(state_slots[b])
        S = state[slot].float().transpose(-1, -2).clone()
        for t in range(cu[b], cu[b + 1]):
            S = d * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
            o[t] = torch.einsum("hdv,hd->hv", S, q[t])
        new[slot] = S.transpose(-1, -2).contiguous()
    return o.view(T, heads * value_dim), new


def ref_headnorm_gate(o, gate, heads, value_dim, eps):
    T = o.shape[0]
    x = o.float().view(T, heads, value_dim)
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return x.reshape(T, heads * value_dim) * torch.nn.functional.silu(gate.float())


_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _mix64(z):
    z = z.astype(np.uint64)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def ref_gumbel(key, vocab):
    """The kernel's noise for one row: key is the row's 64-bit key as a Python int (unsigned)."""
    with np.errstate(over="ignore"):
        i = np.arange(1, vocab + 1, dtype=np.uint64)
        r = _mix64(np.uint64(key) + np.uint64(0x9E3779B97F4A7C15) * i)
    u = ((r >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
    return torch.from_numpy(-np.log(-np.log(u)).astype(np.float32))


def ref_sample(logits, temperature=None, keys=None):
    """Returns (ids, perturbed rows) -- perturbed rows let a test skip near-ties."""
    rows = []
    for r in range(logits.shape[0]):
        row = logits[r].float().cpu()
        T = float(temperature[r]) if temperature is not None else 0.0
        if T > 0:
            key = int(keys[r]) & 0xFFFFFFFFFFFFFFFF
            row = row / T + ref_gumbel(key, row.shape[0])
        rows.append(row)
    rows = torch.stack(rows)
    return rows.argmax(-1).to(torch.int32), rows


class TorchKernels:
    """Same method names and argument order as iitj_llm_coopt_b200.kernels.Kernels."""

    launches = 0

    def embed(self, ids, table, out, scale=1.0):
        out.copy_(ref_embed(ids, table, scale))
        return out

    def add_rmsnorm(self, residual, delta, weight, eps, out, rows=None):
        v, y = ref_add_rmsnorm(residual, delta, weight, eps, rows, out.dtype)
        if rows is None and delta is not None:
            residual.copy_(v)
        out.copy_(y)
        return out

    def rope_tables(self, positions, inv_freq, cos, sin):
        ang = positions.float().unsqueeze(1) * inv_freq.float().unsqueeze(0)
        cos.copy_(ang.cos())
        sin.copy_(ang.sin())
        return cos, sin

    def rope_store(self, qkv, positions, inv_freq, slots, cache_layer, heads, kv_heads, head_dim, rotary_dim, tables=None):
        rot = ref_rope(qkv, positions, inv_freq, heads, kv_heads, head_dim, rotary_dim).to(qkv.dtype)
        if slots is not None:
            ref_store(cache_layer, rot, slots, heads, kv_heads, head_dim)
        qkv[:, :heads * head_dim] = rot[:, :heads * head_dim]
        return qkv

    def silu_mul(self, gu, act):
        act.copy_(ref_silu_mul(gu))
        return act

    def attention(self, qkv, cache_layer, meta, out, heads, kv_heads, head_dim, window=0, scale=0.0):
        out.copy_(ref_paged_attention(qkv, cache_layer, meta.block_table, meta.token_request, meta.positions,
                                      heads, kv_heads, head_dim, window, scale))
        return out

    def linear(self, x, weight, out, swiglu=False, defer=False):
        out.copy_(ref_linear(x, weight, swiglu))     # never split: `defer` has nothing to leave for later
        return out

    def conv_norm_store(self, u, bias, taps_w, q_gain, k_gain, state, state_slots, token_request, cu_seqlens, q_out,
                        cache, slots, heads, kv_heads, head_dim, value_dim, eps):
        own = cache is not None
        q, k, v, new = ref_conv_norm_store(u, bias, taps_w, q_gain, k_gain, state, state_slots, cu_seqlens, heads,
                                           kv_heads, head_dim, value_dim, eps, own)
        q_out.copy_(q)
        if own:
            ps = cache.shape[1] // (kv_heads * (head_dim + value_dim))
            kplane = cache[:, :kv_heads * ps * head_dim].view(-1, kv_heads, ps, head_dim)
            vplane = cache[:, kv_heads * ps * head_dim:].view(-1, kv_heads, ps, value_dim)
            for t in range(u.shape[0]):
                p, o = divmod(int(slots[t]), ps)
                kplane[p, :, o, :] = k[t].view(kv_heads, head_dim).to(cache.dtype)
                vplane[p, :, o, :] = v[t].view(kv_heads, value_dim).to(cache.dtype)
        for slot, rows in new.items():
            state[slot] = rows
        return q_out

    def talking_attention(self, q, cache, meta, talk, slopes, out, heads, kv_heads, head_dim, value_dim, chunk, scale, tiles=None):
        ps = cache.shape[1] // (kv_heads * (head_dim + value_dim))
        out.copy_(ref_talking_attention(q, cache, meta.block_table, meta.token_request, meta.positions, talk, slopes,
                                        heads, kv_heads, head_dim, value_dim, ps, chunk, scale))
        return out

    def retention(self, proj, tables, rotary_dim, decay, state, state_slots, cu_seqlens, o, heads, head_dim, value_dim,
                  k_scale, write=True, longest=0):
        cos, sin = tables if tables is not None else (None, None)
        got, new = ref_retention(proj, cos, sin, rotary_dim, decay, state, state_slots, cu_seqlens, heads, head_dim,
                                 value_dim, k_scale)
        o.copy_(got)
        if write:
            for slot, S in new.items():
                state[slot] = S
        return o

    def headnorm_gate(self, o, proj, gate_col, out, heads, value_dim, eps):
        out.copy_(ref_headnorm_gate(o, proj[:, gate_col:gate_col + heads * value_dim], heads, value_dim, eps))
        return out

    health_codes = (0, 0, 0, 0)     # what `sample` reports as the library's health words (tests set a failure here)

    def scale_(self, x, scale):
        return x.mul_(scale)

    def sample(self, logits, temperature, keys, out, health=None):
        ids, _ = ref_sample(logits, temperature, keys)
        out.copy_(ids)
        if health is not None:
            health[:4] = torch.tensor(self.health_codes, dtype=torch.int32)
        return out

    def check_health(self, codes=None):
        codes = list(self.health_codes if codes is None else codes)
        if any(codes):
            self.health_codes = (0, 0, 0, 0)
            raise RuntimeError(f"a kernel gave up: {codes}")
