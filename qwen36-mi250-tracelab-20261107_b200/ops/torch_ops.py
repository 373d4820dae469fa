"""Plain PyTorch implementations of every engine op.

These are the numerics oracle: each CUDA kernel in ``ops/cuda`` has the same
signature as one function here and is tested against it in fp32 (the reference
keeps a PyTorch twin of each Triton kernel for the same purpose,
``engine/fast/kernels.py:17-21``). They run on any device and dtype; on CPU in
fp32 they are the serving path of the tiny-checkpoint contract tests.

Shapes use packed rows: ``T`` rows of one or more sequences laid end to end.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..config import GDN_CHUNK, PAGE_SIZE


# --------------------------------------------------------------------------- norms
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Zero-centred RMSNorm ``x * rsqrt(mean(x^2)+eps) * (1 + w)`` in fp32, cast back."""
    xf = x.float()
    out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (out * (1.0 + w.float())).to(x.dtype)


def add_rmsnorm(x: torch.Tensor, res: torch.Tensor | None, w: torch.Tensor, eps: float):
    """``res' = res + x`` (rounded to the activation dtype), ``y = rmsnorm(res')``."""
    new = x if res is None else (res + x)
    return new, rmsnorm(new, w, eps)


def gated_rmsnorm(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Per-head ``w * norm(o) * silu(z)`` (plain weight, not zero-centred)."""
    of = o.float()
    n = of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + eps)
    n = (w.float() * n.to(o.dtype).float()) * F.silu(z.float())
    return n.to(o.dtype)


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x @ w.T`` with fp32 accumulation; ``w`` is ``[N, K]``."""
    if out_dtype is not None and out_dtype != x.dtype:
        return (x.float() @ w.float().t()).to(out_dtype)
    return F.linear(x, w)


# --------------------------------------------------------------------------- rope
def rope_cos_sin(positions: torch.Tensor, rotary_dim: int, theta: float):
    """cos/sin ``[T, rotary_dim/2]`` in fp32 for integer positions."""
    inv = 1.0 / (
        theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=positions.device) / rotary_dim)
    )
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def _apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """Rotate the first ``rotary_dim`` dims of ``x [T, heads, D]`` (half-split pairing)."""
    half = rotary_dim // 2
    x1, x2, rest = x[..., :half], x[..., half:rotary_dim], x[..., rotary_dim:]
    c = cos[:, None, :].to(x.dtype)
    s = sin[:, None, :].to(x.dtype)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


# --------------------------------------------------------------------------- attention
def attn_prep(
    qkv: torch.Tensor,
    positions: torch.Tensor,
    q_norm: torch.Tensor,
    k_norm: torch.Tensor,
    n_q: int,
    n_kv: int,
    head_dim: int,
    rotary_dim: int,
    theta: float,
    eps: float,
):
    """Split a merged ``q|gate|k|v`` row, norm q/k per head, apply partial RoPE.

    ``qkv [T, n_q*2*D + 2*n_kv*D]``: the query block holds ``[q | gate]`` per head
    (reference layout: ``engine/fast/model.py:1106-1108``).
    Returns ``q [T,n_q,D]``, ``gate [T,n_q*D]``, ``k [T,n_kv,D]``, ``v [T,n_kv,D]``.
    """
    T = qkv.shape[0]
    qg = qkv[:, : n_q * 2 * head_dim].view(T, n_q, 2 * head_dim)
    q, gate = qg[..., :head_dim], qg[..., head_dim:].reshape(T, n_q * head_dim)
    k = qkv[:, n_q * 2 * head_dim : n_q * 2 * head_dim + n_kv * head_dim].view(T, n_kv, head_dim)
    v = qkv[:, n_q * 2 * head_dim + n_kv * head_dim :].view(T, n_kv, head_dim)
    q = rmsnorm(q, q_norm, eps)
    k = rmsnorm(k, k_norm, eps)
    cos, sin = rope_cos_sin(positions, rotary_dim, theta)
    return _apply_rope(q, cos, sin, rotary_dim), gate, _apply_rope(k, cos, sin, rotary_dim), v


def kv_write(kv_layer: torch.Tensor, k: torch.Tensor, v: torch.Tensor, page_ids: torch.Tensor, offsets: torch.Tensor) -> None:
    """Store rows into the paged cache ``kv_layer [pages, 2, n_kv, PAGE, D]``."""
    kv_layer[page_ids, 0, :, offsets] = k
    kv_layer[page_ids, 1, :, offsets] = v


def _gather_kv(kv_layer: torch.Tensor, table: torch.Tensor, length: int):
    """Contiguous ``k, v [n_kv, length, D]`` of one sequence from its page table."""
    n_pages = (length + PAGE_SIZE - 1) // PAGE_SIZE
    pages = kv_layer[table[:n_pages].long()]  # [n, 2, n_kv, PAGE, D]
    k = pages[:, 0].permute(1, 0, 2, 3).reshape(pages.shape[2], -1, pages.shape[-1])[:, :length]
    v = pages[:, 1].permute(1, 0, 2, 3).reshape(pages.shape[2], -1, pages.shape[-1])[:, :length]
    return k, v


def paged_attention(
    q: torch.Tensor,
    gate: torch.Tensor,
    kv_layer: torch.Tensor,
    block_tables: torch.Tensor,
    seg_starts: list[int],
    seg_pos0: list[int],
) -> torch.Tensor:
    """Causal gated attention of packed query rows against each sequence's paged KV.

    Segment ``i`` owns rows ``seg_starts[i]:seg_starts[i+1]`` at positions
    ``seg_pos0[i]...``; its keys are positions ``0 .. pos0+len`` (already written).
    Returns ``attn * sigmoid(gate)`` as ``[T, n_q*D]``.
    """
    T, n_q, D = q.shape
    n_kv = kv_layer.shape[2]
    group = n_q // n_kv
    out = torch.empty(T, n_q, D, dtype=q.dtype, device=q.device)
    scale = D ** -0.5
    for i in range(len(seg_starts) - 1):
        a, b = seg_starts[i], seg_starts[i + 1]
        n = b - a
        if n == 0:
            continue
        total = seg_pos0[i] + n
        k, v = _gather_kv(kv_layer, block_tables[i], total)
        qs = q[a:b].transpose(0, 1).float()  # [n_q, n, D]
        kf = k.float().repeat_interleave(group, dim=0)
        vf = v.float().repeat_interleave(group, dim=0)
        s = (qs @ kf.transpose(1, 2)) * scale  # [n_q, n, total]
        qpos = torch.arange(seg_pos0[i], total, device=q.device)[:, None]
        kpos = torch.arange(total, device=q.device)[None, :]
        s = s.masked_fill(kpos > qpos, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[a:b] = (p @ vf).transpose(0, 1).to(q.dtype)
    return out.reshape(T, n_q * D) * torch.sigmoid(gate)


# --------------------------------------------------------------------------- MoE
def router_topk(logits: torch.Tensor, top_k: int):
    """fp32 softmax over experts, top-k (ties to the lower id), renormalised weights."""
    probs = torch.softmax(logits.float(), dim=-1)
    # stable descending sort puts the lower expert id first among equal probabilities
    order = torch.sort(probs, dim=-1, descending=True, stable=True)
    vals, idx = order.values[:, :top_k], order.indices[:, :top_k]
    vals = vals / vals.sum(-1, keepdim=True)
    return vals, idx.to(torch.int32)


def moe_experts(
    x: torch.Tensor,
    weights: torch.Tensor,
    idx: torch.Tensor,
    w_gate_up: torch.Tensor,
    w_down: torch.Tensor,
    partial_f32: bool = False,
) -> torch.Tensor:
    """Sum over each row's selected experts of ``w * down(silu(gate(x)) * up(x))``.

    ``weights, idx [T, P]`` (``P`` pairs per row, the shared expert included when it
    is stored as an extra expert), ``w_gate_up [E, 2I, H]``, ``w_down [E, H, I]``.
    Pair outputs are rounded to the activation dtype, then combined in fp32 in pair
    order and rounded once.
    """
    T, P = idx.shape
    inter = w_down.shape[2]
    pair_out = torch.zeros(T, P, x.shape[1], dtype=x.dtype, device=x.device)
    flat = idx.reshape(-1).long()
    for e in torch.unique(flat).tolist():
        if e < 0:
            continue  # hosted by another rank
        sel = (flat == e).nonzero(as_tuple=True)[0]
        rows = sel // P
        gu = linear(x[rows], w_gate_up[e])
        act = F.silu(gu[:, :inter].float()).to(x.dtype) * gu[:, inter:]
        pair_out.view(T * P, -1)[sel] = linear(act, w_down[e])
    out = (pair_out.float() * weights.float()[:, :, None]).sum(1)
    return out if partial_f32 else out.to(x.dtype)


# --------------------------------------------------------------------------- Gated DeltaNet
def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def gdn_gates(a: torch.Tensor, b: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor):
    """``g = -exp(A_log) * softplus(a + dt_bias)`` (log decay) and ``beta = sigmoid(b)``, fp32."""
    g = -A_log.float().exp() * F.softplus(a.float() + dt_bias.float())
    return g, torch.sigmoid(b.float())


def gdn_split(mixed: torch.Tensor, key_dim: int, value_dim: int, n_v: int):
    """Split a merged in_proj row into conv input ``qkv``, ``z``, ``b``, ``a``."""
    conv_dim = 2 * key_dim + value_dim
    qkv = mixed[:, :conv_dim]
    z = mixed[:, conv_dim : conv_dim + value_dim]
    b = mixed[:, conv_dim + value_dim : conv_dim + value_dim + n_v]
    a = mixed[:, conv_dim + value_dim + n_v : conv_dim + value_dim + 2 * n_v]
    return qkv, z, b, a


def causal_conv_prefill(x: torch.Tensor, state: torch.Tensor, w: torch.Tensor):
    """Depthwise causal conv + SiLU over one sequence's rows.

    ``x [n, C]`` new inputs, ``state [C, K-1]`` the previous ``K-1`` inputs, ``w [C, K]``.
    Returns the activations ``[n, C]`` and the new state (last ``K-1`` inputs).
    """
    K = w.shape[1]
    full = torch.cat([state.t().to(x.dtype), x], dim=0)  # [K-1+n, C]
    win = full.unfold(0, K, 1)  # [n, C, K]
    y = (win.float() * w.float()[None]).sum(-1)
    new_state = full[-(K - 1) :].t().contiguous()
    return F.silu(y).to(x.dtype), new_state


def gdn_chunk_rule(q, k, v, g, beta, state, chunk: int = GDN_CHUNK):
    """Chunked gated delta rule over one sequence.

    ``q, k [n, Hv, dk]`` (already L2-normalised, q already scaled), ``v [n, Hv, dv]``,
    ``g, beta [n, Hv]`` fp32, ``state [Hv, dk, dv]`` fp32. Within each chunk the
    strictly-lower system ``(I + A)`` with ``A = (k beta) k^T * exp(g_i - g_j)`` is
    inverted (the WY/UT transform, reference: ``engine/fast/gdn_chunk.py:203-357``);
    chunks are then scanned in order carrying the fp32 state. Padding rows are
    identity (``beta = 0, g = 0``). Returns outputs ``[n, Hv, dv]`` fp32 and the final state.
    """
    n, Hv, dk = k.shape
    dv = v.shape[-1]
    pad = (-n) % chunk
    if pad:
        q = F.pad(q, (0, 0, 0, 0, 0, pad))
        k = F.pad(k, (0, 0, 0, 0, 0, pad))
        v = F.pad(v, (0, 0, 0, 0, 0, pad))
        g = F.pad(g, (0, 0, 0, pad))
        beta = F.pad(beta, (0, 0, 0, pad))
    nc = (n + pad) // chunk
    q, k, v = (t.float().permute(1, 0, 2).reshape(Hv, nc, chunk, -1) for t in (q, k, v))
    g = g.float().t().reshape(Hv, nc, chunk)
    beta = beta.float().t().reshape(Hv, nc, chunk)
    gc = g.cumsum(-1)
    decay = (gc[..., :, None] - gc[..., None, :]).tril().exp().tril()
    kb = k * beta[..., None]
    A = (kb @ k.transpose(-1, -2)) * decay
    A = A.tril(-1)
    eye = torch.eye(chunk, dtype=A.dtype, device=A.device)
    Tinv = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False, unitriangular=True)
    u = Tinv @ (v * beta[..., None])
    w = Tinv @ (kb * gc.exp()[..., None])
    qk = ((q @ k.transpose(-1, -2)) * decay).tril()
    out = torch.empty(Hv, nc, chunk, dv, dtype=torch.float32, device=q.device)
    S = state.float().clone()
    for c in range(nc):
        v_new = u[:, c] - w[:, c] @ S
        out[:, c] = (q[:, c] * gc[:, c].exp()[..., None]) @ S + qk[:, c] @ v_new
        last = gc[:, c, -1]
        S = S * last.exp()[:, None, None] + (k[:, c] * (last[:, None] - gc[:, c]).exp()[..., None]).transpose(
            -1, -2
        ) @ v_new
    out = out.reshape(Hv, nc * chunk, dv)[:, :n].permute(1, 0, 2)
    return out, S


def gdn_recurrent_step(q, k, v, g, beta, state):
    """One token of the gated delta rule for a batch: state ``[B, Hv, dk, dv]`` fp32, in place.

    ``S *= exp(g)``; ``kv = S^T k``; ``S += k (beta (v - kv))^T``; ``o = S^T q``
    (reference: ``engine/fast/kernels.py:597-633``).
    """
    S = state * g.exp()[..., None, None]
    kv = (S * k[..., None]).sum(-2)
    delta = (v - kv) * beta[..., None]
    S = S + k[..., None] * delta[..., None, :]
    o = (S * q[..., None]).sum(-2)
    state.copy_(S)
    return o


def _gdn_qkv_heads(conv_out: torch.Tensor, n_k: int, n_v: int, dk: int, dv: int):
    key_dim = n_k * dk
    T = conv_out.shape[0]
    q = conv_out[:, :key_dim].view(T, n_k, dk)
    k = conv_out[:, key_dim : 2 * key_dim].view(T, n_k, dk)
    v = conv_out[:, 2 * key_dim :].view(T, n_v, dv)
    rep = n_v // n_k
    q = l2norm(q.float()) * (dk ** -0.5)
    k = l2norm(k.float())
    if rep > 1:
        q = q.repeat_interleave(rep, dim=1)
        k = k.repeat_interleave(rep, dim=1)
    return q, k, v.float()


def gdn_prefill(
    mixed: torch.Tensor,
    seg_starts: list[int],
    seg_slots: list[int],
    conv_state: torch.Tensor,
    rec_state: torch.Tensor,
    conv_w: torch.Tensor,
    A_log: torch.Tensor,
    dt_bias: torch.Tensor,
    gnorm_w: torch.Tensor,
    n_k: int,
    n_v: int,
    dk: int,
    dv: int,
    eps: float,
) -> torch.Tensor:
    """Gated DeltaNet mixer over packed prefill rows; updates each segment's slot state.

    ``mixed [T, qkv|z|b|a]``; ``conv_state [slots, C, K-1]``; ``rec_state [slots, Hv, dk, dv]``.
    Returns the gated-normed core output ``[T, Hv*dv]``.
    """
    qkv, z, b, a = gdn_split(mixed, n_k * dk, n_v * dv, n_v)
    g_all, beta_all = gdn_gates(a, b, A_log, dt_bias)
    out = torch.empty(mixed.shape[0], n_v, dv, dtype=mixed.dtype, device=mixed.device)
    for i in range(len(seg_starts) - 1):
        s, e = seg_starts[i], seg_starts[i + 1]
        if s == e:
            continue
        slot = seg_slots[i]
        conv_out, new_conv = causal_conv_prefill(qkv[s:e], conv_state[slot], conv_w)
        conv_state[slot] = new_conv.to(conv_state.dtype)
        q, k, v = _gdn_qkv_heads(conv_out, n_k, n_v, dk, dv)
        o, S = gdn_chunk_rule(q, k, v, g_all[s:e], beta_all[s:e], rec_state[slot])
        rec_state[slot] = S
        out[s:e] = o.to(mixed.dtype)
    zz = z.reshape(-1, n_v, dv)
    return gated_rmsnorm(out, zz, gnorm_w, eps).reshape(mixed.shape[0], n_v * dv)


def gdn_decode(
    mixed: torch.Tensor,
    slots: torch.Tensor,
    conv_state: torch.Tensor,
    rec_state: torch.Tensor,
    conv_w: torch.Tensor,
    A_log: torch.Tensor,
    dt_bias: torch.Tensor,
    gnorm_w: torch.Tensor,
    n_k: int,
    n_v: int,
    dk: int,
    dv: int,
    eps: float,
    G: int = 1,
    ring=None,
) -> torch.Tensor:
    """Decode rows: conv step, recurrent delta rule, gated norm; slot state updated in place.

    ``mixed [B*G, .]`` holds ``G`` consecutive rows per slot (``G = 1`` plain decode, ``G = k+1``
    speculative verify), processed in order. With ``ring = (conv [B,G,C,K-1], rec [B,G,Hv,dk,dv])``
    the state after every row is also stored, so that a verify step can commit any prefix.
    """
    rows = mixed.shape[0]
    B = rows // G
    qkv_all, z_all, b_all, a_all = gdn_split(mixed, n_k * dk, n_v * dv, n_v)
    g_all, beta_all = gdn_gates(a_all, b_all, A_log, dt_bias)
    sl = slots.long()
    out = torch.empty(rows, n_v * dv, dtype=mixed.dtype, device=mixed.device)
    base = torch.arange(B, device=mixed.device) * G
    conv = conv_state[sl].to(mixed.dtype)
    S = rec_state[sl].clone()
    for j in range(G):
        r = base + j
        win = torch.cat([conv, qkv_all[r][:, :, None]], dim=-1)  # [B, C, K]
        conv_out = F.silu((win.float() * conv_w.float()[None]).sum(-1)).to(mixed.dtype)
        conv = win[:, :, 1:]
        q, k, v = _gdn_qkv_heads(conv_out, n_k, n_v, dk, dv)
        o = gdn_recurrent_step(q, k, v, g_all[r], beta_all[r], S)
        out[r] = gated_rmsnorm(o.to(mixed.dtype), z_all[r].reshape(B, n_v, dv), gnorm_w, eps).reshape(B, n_v * dv)
        if ring is not None:
            ring[0][:, j] = conv.to(ring[0].dtype)
            ring[1][:, j] = S
    conv_state[sl] = conv.to(conv_state.dtype)
    rec_state[sl] = S
    return out


def gdn_prefill_batched(
    mixed, seg_starts, seg_slots, conv_state, rec_state, conv_w, A_log, dt_bias, gnorm_w, n_k, n_v, dk, dv, eps,
    chunk: int = GDN_CHUNK,
) -> torch.Tensor:
    """``gdn_prefill`` vectorised over sequences: spans are padded to a common chunk count with
    identity rows (``beta = 0``, ``g = 0``, zero inputs), which leave the state untouched."""
    dev = mixed.device
    T = mixed.shape[0]
    nseg = len(seg_slots)
    lens = [seg_starts[i + 1] - seg_starts[i] for i in range(nseg)]
    Lmax = max(lens)
    Lp = (Lmax + chunk - 1) // chunk * chunk
    nc = Lp // chunk
    K = conv_w.shape[1]
    qkv, z, b, a = gdn_split(mixed, n_k * dk, n_v * dv, n_v)
    g_all, beta_all = gdn_gates(a, b, A_log, dt_bias)
    # row r of segment i sits at padded index (i, r - start_i)
    seg_of_row = torch.repeat_interleave(torch.arange(nseg, device=dev), torch.tensor(lens, device=dev))
    starts = torch.tensor(seg_starts[:-1], device=dev)
    off = torch.arange(T, device=dev) - starts[seg_of_row]
    slots = torch.tensor(seg_slots, device=dev)
    lens_t = torch.tensor(lens, device=dev)
    C = qkv.shape[1]
    xin = torch.zeros(nseg, K - 1 + Lp, C, dtype=mixed.dtype, device=dev)
    xin[:, : K - 1] = conv_state[slots].transpose(1, 2).to(mixed.dtype)
    xin[seg_of_row, off + K - 1] = qkv
    win = xin.unfold(1, K, 1)  # [nseg, Lp, C, K]
    conv_out = F.silu((win.float() * conv_w.float()[None, None]).sum(-1)).to(mixed.dtype)
    tail_idx = lens_t[:, None] + torch.arange(K - 1, device=dev)[None, :]  # last K-1 inputs of each span
    conv_state[slots] = torch.gather(xin, 1, tail_idx[:, :, None].expand(-1, -1, C)).transpose(1, 2).to(conv_state.dtype)
    q, k, v = _gdn_qkv_heads(conv_out.reshape(nseg * Lp, C), n_k, n_v, dk, dv)
    valid = (torch.arange(Lp, device=dev)[None, :] < lens_t[:, None]).reshape(nseg * Lp, 1, 1)
    q, k, v = q * valid, k * valid, v * valid
    g = torch.zeros(nseg, Lp, n_v, dtype=torch.float32, device=dev)
    beta = torch.zeros(nseg, Lp, n_v, dtype=torch.float32, device=dev)
    g[seg_of_row, off] = g_all
    beta[seg_of_row, off] = beta_all
    # [nseg, Hv, nc, chunk, d]
    q, k, v = (t.view(nseg, Lp, n_v, -1).permute(0, 2, 1, 3).reshape(nseg, n_v, nc, chunk, -1) for t in (q, k, v))
    g = g.permute(0, 2, 1).reshape(nseg, n_v, nc, chunk)
    beta = beta.permute(0, 2, 1).reshape(nseg, n_v, nc, chunk)
    gc = g.cumsum(-1)
    decay = (gc[..., :, None] - gc[..., None, :]).tril().exp().tril()
    kb = k * beta[..., None]
    A = ((kb @ k.transpose(-1, -2)) * decay).tril(-1)
    eye = torch.eye(chunk, dtype=A.dtype, device=dev)
    Tinv = torch.linalg.solve_triangular(eye + A, eye.expand_as(A).contiguous(), upper=False, unitriangular=True)
    u = Tinv @ (v * beta[..., None])
    w = Tinv @ (kb * gc.exp()[..., None])
    qk = ((q @ k.transpose(-1, -2)) * decay).tril()
    out = torch.empty(nseg, n_v, nc, chunk, dv, dtype=torch.float32, device=dev)
    S = rec_state[slots].float().clone()
    for c in range(nc):
        v_new = u[:, :, c] - w[:, :, c] @ S
        out[:, :, c] = (q[:, :, c] * gc[:, :, c].exp()[..., None]) @ S + qk[:, :, c] @ v_new
        last = gc[:, :, c, -1]
        S = S * last.exp()[..., None, None] + (
            k[:, :, c] * (last[..., None] - gc[:, :, c]).exp()[..., None]
        ).transpose(-1, -2) @ v_new
    rec_state[slots] = S
    o = out.reshape(nseg, n_v, Lp, dv).permute(0, 2, 1, 3)[seg_of_row, off]  # [T, Hv, dv]
    return gated_rmsnorm(o.to(mixed.dtype), z.reshape(T, n_v, dv), gnorm_w, eps).reshape(T, n_v * dv)


# --------------------------------------------------------------------------- composite blocks
def embed(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    return table[tokens]


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    inter = w_gate_up.shape[0] // 2
    gu = linear(x, w_gate_up)
    return F.silu(gu[:, :inter].float()).to(x.dtype) * gu[:, inter:]


def lm_head_argmax(x: torch.Tensor, w: torch.Tensor, return_value: bool = False):
    logits = linear(x, w, out_dtype=torch.float32)
    idx = argmax_rows(logits)
    if return_value:
        return idx, logits.gather(1, idx[:, None])[:, 0]
    return idx


def moe_block(x, router, w_gate_up, w_down, n_experts: int, top_k: int, shared_merged: bool,
              expert_map: torch.Tensor | None = None, partial_f32: bool = False) -> torch.Tensor:
    """Router, top-k and experts; with ``shared_merged`` router row ``E`` is the shared gate and
    expert ``E`` the shared expert, selected for every row with weight ``sigmoid(logit_E)``.

    ``expert_map`` (global id -> local slot or -1) restricts the work to locally hosted experts;
    ``partial_f32`` returns the unrounded fp32 partial sum for a cross-rank reduction."""
    logits = linear(x, router, out_dtype=torch.float32)
    wts, idx = router_topk(logits[:, :n_experts], top_k)
    if shared_merged:
        wts = torch.cat([wts, torch.sigmoid(logits[:, n_experts : n_experts + 1])], dim=1)
        idx = torch.cat([idx, torch.full_like(idx[:, :1], n_experts)], dim=1)
    wts = wts.to(x.dtype)
    if expert_map is not None:
        local = expert_map.to(idx.device)[idx.long()]
        wts = torch.where(local >= 0, wts, torch.zeros_like(wts))
        idx = local
    return moe_experts(x, wts, idx, w_gate_up, w_down, partial_f32=partial_f32)


def attention(qkv, positions, seq_of_row, block_tables, kv_layer, q_norm, k_norm, n_q, n_kv, head_dim, rotary_dim,
              theta, eps, G: int, seg_starts=None, seg_pos0=None) -> torch.Tensor:
    """q/k norm, RoPE, KV page write and causal gated attention over the paged cache (see ``cuda_ops.attention``)."""
    q, gate, k, v = attn_prep(qkv, positions, q_norm, k_norm, n_q, n_kv, head_dim, rotary_dim, theta, eps)
    page_ids = block_tables[seq_of_row.long(), positions // PAGE_SIZE].long()
    kv_write(kv_layer, k, v, page_ids, positions % PAGE_SIZE)
    if G > 0:
        B = qkv.shape[0] // G
        seg_starts = [i * G for i in range(B + 1)]
        seg_pos0 = positions[::G].tolist()
    return paged_attention(q, gate, kv_layer, block_tables, seg_starts, seg_pos0)


# --------------------------------------------------------------------------- head
def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """First index of the row maximum (ties to the lower id)."""
    return torch.argmax(logits.float(), dim=-1)


def softplus_inv(x: float) -> float:
    return math.log(math.expm1(x))
