"""Plain PyTorch float32 statements of what each kernel of ``inferrs_b200.kernels`` computes.

Same names and arguments as the kernels; they work on any device.  The GPU
tests compare every kernel with its function here; the CPU tests put these in
the kernels' place (``install``) to exercise the engine's own logic (cache,
batches, steps) on a machine without a GPU.  They are slow on purpose: loops
over rows, no cleverness.
"""
from __future__ import annotations

from typing import Optional

import torch


def embedding_gather(table, ids, out, act_dtype=None, scale=1.0):
    out.copy_(table[ids.long()].float() * scale)


def rms_norm_rows(x, weight, eps, out):
    v = x.float()
    out.copy_((v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps) * weight.float()).to(out.dtype))


def add_cast(residual, delta, out, rows=None):
    if rows is None:
        if delta is not None:
            residual += delta.float()
        out.copy_(residual.to(out.dtype))
    else:
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
        out.copy_(x.to(out.dtype))


def logit_scale_softcap(logits, scale, softcap, act_dtype=None):
    logits.mul_(scale)
    if softcap:
        logits.copy_(softcap * torch.tanh(logits / softcap))


def add_rms_norm(residual, delta, weight, eps, out, rows=None):
    if rows is None:
        if delta is not None:
            residual += delta.float()
        x = residual
    else:
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    ms = (x * x).mean(dim=-1, keepdim=True)
    out.copy_((x / torch.sqrt(ms + eps) * weight.float()).to(out.dtype))


def silu_gate(gate_up, out):
    inner = out.shape[1]
    g, u = gate_up[:, :inner].float(), gate_up[:, inner:].float()
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def _rms(x, w, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w.float()


def _rotate(x, cos, sin, rot_dim, interleaved=False):
    # x [rows, heads, d]; cos/sin [rows, rot_dim/2]
    half = rot_dim // 2
    if interleaved:
        x1, x2, rest = x[..., 0:rot_dim:2], x[..., 1:rot_dim:2], x[..., rot_dim:]
        c, s = cos[:, None, :], sin[:, None, :]
        turned = torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1).flatten(-2)
        return torch.cat([turned, rest], dim=-1)
    x1, x2, rest = x[..., :half], x[..., half:rot_dim], x[..., rot_dim:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c, rest], dim=-1)


def qk_norm_rope_store(qkv, n_heads, n_kv_heads, head_dim, store_kv, q_weight, k_weight, eps, cos, sin, rot_dim,
                       positions, row_request, block_table, k_pages, v_pages, q_out, interleaved=False):
    n = qkv.shape[0]
    d = head_dim
    x = qkv.float()
    q = x[:, :n_heads * d].reshape(n, n_heads, d)
    pos = positions.long()
    if q_weight is not None:
        q = _rms(q, q_weight, eps)
    if rot_dim:
        q = _rotate(q, cos[pos], sin[pos], rot_dim, interleaved)
    q_out.copy_(q.to(q_out.dtype))
    if not store_kv:
        return
    k = x[:, n_heads * d:(n_heads + n_kv_heads) * d].reshape(n, n_kv_heads, d)
    v = x[:, (n_heads + n_kv_heads) * d:].reshape(n, n_kv_heads, d)
    if k_weight is not None:
        k = _rms(k, k_weight, eps)
    if rot_dim:
        k = _rotate(k, cos[pos], sin[pos], rot_dim, interleaved)
    page_size = k_pages.shape[2]
    for r in range(n):
        p = int(positions[r])
        page = int(block_table[int(row_request[r]), p // page_size])
        assert page >= 0, "a row writes into a page that was given back"
        k_pages[page, :, p % page_size, :] = k[r].to(k_pages.dtype)
        v_pages[page, :, p % page_size, :] = v[r].to(v_pages.dtype)
        if r + 1 == n or int(row_request[r + 1]) != int(row_request[r]):
            # a request's last row clears the places behind its value in the page (kernels that fetch whole pages
            # multiply them by a probability of zero)
            v_pages[page, :, p % page_size + 1:, :] = 0


def paged_attention_generic(q, k_pages, v_pages, block_table, row_request, positions, scale, window, out):
    n, nh, d = q.shape
    nkv, page_size = k_pages.shape[1], k_pages.shape[2]
    g = nh // nkv
    for r in range(n):
        pos = int(positions[r])
        req = int(row_request[r])
        lo = max(0, pos - window + 1) if window else 0
        js = torch.arange(lo, pos + 1)
        pages = block_table[req, (js // page_size).long()].long()
        assert (pages >= 0).all(), "a visible key lies in a page that was given back"
        k = k_pages[pages, :, (js % page_size).long(), :].float()  # [keys, nkv, d]
        v = v_pages[pages, :, (js % page_size).long(), :].float()
        k = k.repeat_interleave(g, dim=1)
        v = v.repeat_interleave(g, dim=1)
        s = torch.einsum("hd,khd->hk", q[r].float(), k) * scale
        p = torch.softmax(s, dim=-1)
        o = torch.einsum("hk,khd->hd", p, v)
        out[r] = o.reshape(nh * d).to(out.dtype)


def paged_attention(q, k_pages, v_pages, block_table, ctx, scale, window, out):
    paged_attention_generic(q, k_pages, v_pages, block_table, ctx.row_request, ctx.positions, scale, window, out)


def gemm_tn_simt(x, w, out, act_dtype=None):
    out.copy_((x.float() @ w.float().t()).to(out.dtype))


def gemm_tn_bf16(x, w, out):
    out.copy_((x.float() @ w.float().t()).to(out.dtype))


def _unscale(x):
    """What scaled rows stand for: (stream * weight) / sqrt(sum of squares / width + eps) per row."""
    ss = x.ssq[:x.n_parts, :x.x.shape[0]].sum(dim=0)
    return x.x.float() / torch.sqrt(ss / x.width + x.eps)[:, None]


def linear(x, w, out, act_dtype=None, sink=None):
    """With scaled rows and a sink as the product with folded norms defines them (csrc/gemm_tcgen05.cu)."""
    import inferrs_b200.kernels as K
    xf = _unscale(x) if isinstance(x, K.ScaledRows) else x.float()
    y = xf @ w.float().t()
    if sink is None:
        out.copy_(y.to(out.dtype))
        return None
    sink.residual += y.to(out.dtype).float()
    out.copy_((sink.residual * sink.weight.float()).to(out.dtype))
    ssq = torch.zeros((1, K.SSQ_LD), dtype=torch.float32, device=out.device)
    ssq[0, :out.shape[0]] = (sink.residual * sink.residual).sum(dim=1)
    return K.ScaledRows(out, ssq, 1, float(sink.eps), out.shape[1])


def gated_linear(x, w_gate_up, out, act_dtype=None):
    import inferrs_b200.kernels as K
    xf = _unscale(x) if isinstance(x, K.ScaledRows) else x.float()
    gu = (xf @ w_gate_up.float().t()).to(out.dtype)
    silu_gate(gu, out)


def argmax(logits, out, act_dtype=None):
    out.copy_(torch.argmax(logits, dim=-1).to(out.dtype))


_NAMES = ["embedding_gather", "add_rms_norm", "silu_gate", "qk_norm_rope_store", "paged_attention_generic",
          "paged_attention", "gemm_tn_simt", "gemm_tn_bf16", "linear", "gated_linear", "argmax"]


def install(monkeypatch):
    """Put the plain functions in the kernels' place for one test (a pytest ``monkeypatch``)."""
    import inferrs_b200.kernels as K

    for name in _NAMES:
        monkeypatch.setattr(K, name, globals()[name])


def penalties(logits, prev, n_prev, repetition, frequency, presence, act_dtype=None):
    for r in range(logits.shape[0]):
        window = [int(t) for t in prev[r, :int(n_prev[r])]]
        rp, fp, pp = float(repetition[r]), float(frequency[r]), float(presence[r])
        for t in dict.fromkeys(window):
            if not 0 <= t < logits.shape[1]:
                continue
            v = logits[r, t]
            if rp not in (1.0, 0.0):
                v = v / rp if v >= 0 else v * rp
            if fp != 0.0 or pp != 0.0:
                v = v - fp * window.count(t) - pp
            logits[r, t] = v


def sample(logits, temperature, top_k, top_p, min_p, uniform, out, act_dtype=None, cluster=0):
    for r in range(logits.shape[0]):
        t = float(temperature[r])
        if t < 1e-5:
            out[r] = int(torch.argmax(logits[r]))
            continue
        z = logits[r].float() / t
        e = torch.exp(z - z.max()).double()
        order = torch.sort(e, descending=True, stable=True).indices
        total = e.sum()
        k = int(top_k[r])
        if 0 < k < len(order):
            order = order[:k]
        cum = torch.cumsum(e[order], 0)
        if float(top_p[r]) < 1.0:
            hit = (cum >= float(top_p[r]) * total).nonzero()
            if len(hit):
                order = order[:int(hit[0]) + 1]
        if float(min_p[r]) > 0.0:
            keep = int((e[order] >= float(min_p[r])).sum())
            if keep > 0:
                order = order[:keep]
        cum = torch.cumsum(e[order], 0)
        target = float(uniform[r]) * float(cum[-1])
        hit = (cum > target).nonzero()
        out[r] = int(order[int(hit[0])]) if len(hit) else int(order[-1])


_NAMES += ["penalties", "sample", "rms_norm_rows", "add_cast", "logit_scale_softcap"]
