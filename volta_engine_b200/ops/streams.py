"""Multi-stream residual modules: hyper-connections, gated residual streams, the n-gram embedding layer's device side and
the row epilogues that follow a row-parallel projection (sandwich norm, gated stream update, hyper-connection update).

Every function takes CUDA tensors (kernels of csrc/cuda/streams.cu, or the fused all-reduce of csrc/cuda/comm.cu when the
communicator offers it and the rows fit) or CPU tensors (the fp32 PyTorch statement of the same arithmetic, which is also
the oracle of the kernel tests).

Reference: inc/engine/modules/mhc.h + src/kernels/slang/mhc.slang (hyper-connections), inc/engine/modules/gated_residual.h +
src/backend/cpu/gated_residual.cpp, inc/engine/modules/ple.h + src/backend/cpu/ple.cpp, and the fused all-reduce forms of
src/comm/all_reduce_ipc.cu:404-768.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .._lib import call, ptr

PLE_RING = 16
EPI_SANDWICH, EPI_GATED, EPI_HC = 2, 3, 4
_EPI_SIG = "ipl" + "p" * 10 + "iiifff"
LL_EPI_SIG = "piipl" + "p" * 10 + "iiifff"


def _bf(x):
    return x.to(torch.bfloat16).float()


def _p(t):
    return ptr(t) if t is not None else 0


# ---------------------------------------------------------------------------------------------- row epilogues
def _fused_rows_ok(comm, part) -> bool:
    return comm is not None and getattr(comm, "size", 1) > 1 and hasattr(comm, "allreduce_epilogue") and part.is_cuda and \
        part.shape[0] <= 16


def _reduce(comm, part):
    if comm is None or getattr(comm, "size", 1) == 1:
        return part
    return comm.allreduce_(part)


def _epilogue(mode, comm, part, *, xs=None, res16=None, post=None, comb=None, w=None, w2=None, addend=None, addend_gate=None,
              out=None, outf=None, hc=1, eps=1e-6, wbias=0.0, scale=1.0):
    rows, H = part.shape
    args = (_p(xs), _p(res16), _p(post), _p(comb), _p(w), _p(w2), _p(addend), _p(addend_gate), _p(out), _p(outf), rows, H, hc,
            float(eps), float(wbias), float(scale))
    if _fused_rows_ok(comm, part):
        comm.allreduce_epilogue(mode, part, args)
        return
    y = _reduce(comm, part)
    call("stream_epilogue", _EPI_SIG, mode, ptr(y), y.stride(0), *args)


def sandwich_add_norm(part, resid, w_post, w_next, eps, wbias=0.0, scale=1.0, comm=None, out=None):
    """resid = (resid + RMSNorm(sum_ranks part) * (w_post + b)) * scale, in place (fp32 or bf16 residual);
    returns RMSNorm(resid) * (w_next + b) in bf16."""
    if not part.is_cuda:
        y = _bf(_reduce(comm, part).float())
        t = _bf(y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * (w_post.float() + wbias))
        r = (resid.float() + t) * scale
        if resid.dtype != torch.float32:
            r = _bf(r)
        resid.copy_(r)
        return (r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + eps) * (w_next.float() + wbias)).to(torch.bfloat16)
    if out is None:
        out = torch.empty(part.shape, dtype=torch.bfloat16, device=part.device)
    f32 = resid.dtype == torch.float32
    _epilogue(EPI_SANDWICH, comm, part, xs=resid if f32 else None, res16=None if f32 else resid, w=w_post, w2=w_next, out=out,
              eps=eps, wbias=wbias, scale=scale)
    return out


def gated_stream_update(part, streams, post, norm_w=None, eps=1e-6, addend=None, addend_gate=None, comm=None, out_dtype=None):
    """streams[r, s] += post[r, s] * (sum_ranks part[r] [+ addend_gate[r] * addend[r]]), in place; with ``norm_w`` [hc, H] also
    returns the per-stream RMSNorm(streams) * (1 + norm_w) as ``out_dtype`` (float32: the next mixer's input; bfloat16)."""
    rows, hc, H = streams.shape
    out_dtype = out_dtype or torch.float32
    if not part.is_cuda:
        y = _bf(_reduce(comm, part).float())
        if addend is not None:
            y = _bf(y + addend_gate.float()[:, None] * addend.float())
        streams += post[:, :, None] * y[:, None, :]
        if norm_w is None:
            return None
        n = streams * torch.rsqrt(streams.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + norm_w.float())[None]
        return n.to(out_dtype)
    out = None
    if norm_w is not None:
        out = torch.empty(rows, hc, H, dtype=out_dtype, device=part.device)
    _epilogue(EPI_GATED, comm, part, xs=streams, post=post, w=norm_w, addend=addend, addend_gate=addend_gate,
              out=out if out_dtype == torch.bfloat16 else None, outf=out if out_dtype == torch.float32 else None, hc=hc, eps=eps)
    return out


def hc_update(part, streams, post, comb, comm=None):
    """streams[r, h] = post[r, h] * y[r] + sum_g comb[r, g, h] * streams[r, g] with y = sum_ranks part, in place (4 streams)."""
    if not part.is_cuda:
        y = _bf(_reduce(comm, part).float())
        new = post[:, :, None] * y[:, None, :] + torch.einsum("rgh,rgd->rhd", comb, streams)
        streams.copy_(new)
        return streams
    _epilogue(EPI_HC, comm, part, xs=streams, post=post, comb=comb, hc=4)
    return streams


# ---------------------------------------------------------------------------------------------- shared small kernels
def init_streams(x, hc):
    rows, H = x.shape
    if not x.is_cuda:
        return x.float()[:, None, :].repeat(1, hc, 1).contiguous()
    xs = torch.empty(rows, hc, H, dtype=torch.float32, device=x.device)
    call("init_streams", "ppiii", ptr(x), ptr(xs), rows, H, hc)
    return xs


def head_mean(streams):
    rows, hc, H = streams.shape
    if not streams.is_cuda:
        return (streams.sum(1) / hc).to(torch.bfloat16)
    out = torch.empty(rows, H, dtype=torch.bfloat16, device=streams.device)
    call("head_mean", "ppiii", ptr(streams), ptr(out), rows, H, hc)
    return out


def add_broadcast(h, e, hc):
    """streams[r, s] = h[r * hc + s] + e[r]."""
    rows, H = e.shape
    if not h.is_cuda:
        return h.float().reshape(rows, hc, H) + e.float()[:, None, :]
    xs = torch.empty(rows, hc, H, dtype=torch.float32, device=h.device)
    call("add_broadcast", "pppiii", ptr(h), ptr(e), ptr(xs), rows, H, hc)
    return xs


# ---------------------------------------------------------------------------------------------- hyper-connections
@dataclass
class HcMix:
    collapsed: torch.Tensor      # [rows, D] bf16 (normalised when a norm weight was given)
    post: torch.Tensor           # [rows, 4]
    comb: torch.Tensor           # [rows, 4, 4]
    pre: torch.Tensor            # [rows, 4]
    inv_rms: torch.Tensor        # [rows]
    mix_logits: torch.Tensor     # [rows, 24]


def hc_collapse(streams, fn, base, scale, iters=20, hc_eps=1e-6, rms_eps=1e-5, norm_w=None, norm_eps=1e-6, norm_bias=0.0,
                pre_in=None, post_scale=1.0) -> HcMix:
    """The hyper-connection read step for fp32 streams [rows, 4, D]: mix logits against ``fn`` [24, 4*D], the three gates and
    the collapsed row; ``norm_w`` adds the RMSNorm of the collapsed row, ``pre_in`` [rows, 4] collapses with the previous
    step's gate (the lagged form), ``post_scale`` multiplies post."""
    rows, _, D = streams.shape
    dev = streams.device
    if not streams.is_cuda:
        flat = streams.reshape(rows, 4 * D)
        mix = flat @ fn.t()
        rmr = torch.rsqrt(flat.pow(2).sum(-1) / (4 * D) + rms_eps)
        z = mix * rmr[:, None]
        pre = torch.sigmoid(z[:, 0:4] * scale[0] + base[0:4]) + hc_eps
        post = 2.0 * torch.sigmoid(z[:, 4:8] * scale[1] + base[4:8]) * post_scale
        v = torch.softmax((z[:, 8:24] * scale[2] + base[8:24]).reshape(rows, 4, 4), dim=-1) + hc_eps
        v = v / (v.sum(1, keepdim=True) + hc_eps)
        for _ in range(iters - 1):
            v = v / (v.sum(2, keepdim=True) + hc_eps)
            v = v / (v.sum(1, keepdim=True) + hc_eps)
        use = pre if pre_in is None else pre_in
        col = _bf(torch.einsum("rh,rhd->rd", use, streams))
        if norm_w is not None:
            col = col * torch.rsqrt(col.pow(2).mean(-1, keepdim=True) + norm_eps) * (norm_w.float() + norm_bias)
        return HcMix(col.to(torch.bfloat16), post, v, pre, rmr, mix)
    col = torch.empty(rows, D, dtype=torch.bfloat16, device=dev)
    post = torch.empty(rows, 4, dtype=torch.float32, device=dev)
    comb = torch.empty(rows, 4, 4, dtype=torch.float32, device=dev)
    pre = torch.empty(rows, 4, dtype=torch.float32, device=dev)
    inv = torch.empty(rows, dtype=torch.float32, device=dev)
    logits = torch.empty(rows, 24, dtype=torch.float32, device=dev)
    call("hc_collapse", "pppppppppppp" + "iii" + "fffff", ptr(streams), ptr(fn), ptr(base), ptr(scale), _p(pre_in), _p(norm_w),
         ptr(col), ptr(post), ptr(comb), ptr(inv), ptr(logits), ptr(pre), rows, D, iters, float(hc_eps), float(rms_eps),
         float(norm_eps), float(norm_bias), float(post_scale))
    return HcMix(col, post, comb, pre, inv, logits)


# ---------------------------------------------------------------------------------------------- gated residual
@dataclass
class GatedResidualWeights:
    norm: torch.Tensor           # [hc, H] bf16, applied as 1 + w
    down: torch.Tensor           # [rank, hc * H] bf16
    up: torch.Tensor             # [hc * H, rank] bf16
    inject: torch.Tensor | None  # [hc, hc * H] bf16 (absent on the final mixer)

    @property
    def rank(self):
        return self.down.shape[0]


def gr_norm(streams, norm_w, eps, prev_post=None, prev_y=None, want_split=False):
    """Per-stream RMSNorm * (1 + w) of fp32 streams, after folding in a deferred ``streams += prev_post * prev_y``.
    Returns normed fp32 [rows, hc, H] (and its bf16 hi / lo halves with ``want_split``)."""
    rows, hc, H = streams.shape
    if not streams.is_cuda:
        if prev_y is not None:
            streams += prev_post[:, :, None] * prev_y.float()[:, None, :]
        n = streams * torch.rsqrt(streams.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + norm_w.float())[None]
        if want_split:
            hi = n.to(torch.bfloat16)
            return n, hi, (n - hi.float()).to(torch.bfloat16)
        return n
    n = torch.empty_like(streams)
    hi = lo = None
    if want_split:
        hi = torch.empty(rows, hc, H, dtype=torch.bfloat16, device=streams.device)
        lo = torch.empty_like(hi)
    call("gr_norm", "pppppppiiif", ptr(streams), ptr(norm_w), ptr(n), _p(hi), _p(lo), _p(prev_post), _p(prev_y), rows, H, hc,
         float(eps))
    return (n, hi, lo) if want_split else n


def gr_mix_prenormed(normed, W: GatedResidualWeights, gemm_rows: int = 64):
    """(mixed bf16 [rows, H], post fp32 [rows, hc] or None) from the normalised streams. Rows up to ``gemm_rows`` stream
    the gate weights through the mat-vec kernels; more rows take the tensor-core GEMM with the fp32 operand split into
    bf16 hi + lo halves (two GEMMs accumulated in fp32)."""
    rows, hc, H = normed.shape
    rank = W.rank
    if not normed.is_cuda:
        flat = normed.reshape(rows, hc * H)
        z = flat @ W.down.float().t() / hc
        t = z * torch.sigmoid(z)
        post = 2.0 * torch.sigmoid(flat @ W.inject.float().t() / hc) if W.inject is not None else None
        u = (t @ W.up.float().t()).reshape(rows, hc, H)
        return ((torch.sigmoid(u) * normed).sum(1) / hc).to(torch.bfloat16), post
    dev = normed.device
    mixed = torch.empty(rows, H, dtype=torch.bfloat16, device=dev)
    post = torch.empty(rows, hc, dtype=torch.float32, device=dev) if W.inject is not None else None
    if rows <= gemm_rows:
        t = torch.empty(rows, rank, dtype=torch.float32, device=dev)
        call("gr_gate", "pppppiiii", ptr(normed), ptr(W.down), _p(W.inject), ptr(t), _p(post), rows, H, hc, rank)
        call("gr_up", "ppppiiii", ptr(normed), ptr(t), ptr(W.up), ptr(mixed), rows, H, hc, rank)
        return mixed, post
    from . import kernels as K
    flat = normed.reshape(rows, hc * H)
    hi = flat.to(torch.bfloat16)
    lo = (flat - hi.float()).to(torch.bfloat16)
    wcat = W.down if W.inject is None else torch.cat([W.down, W.inject], 0)
    z = (K.gemm_bf16(wcat, hi, out_f32=True) + K.gemm_bf16(wcat, lo, out_f32=True)) / hc
    zt = z[:, :rank]
    t = zt * torch.sigmoid(zt)
    if post is not None:
        post.copy_(2.0 * torch.sigmoid(z[:, rank:rank + hc]))
    thi = t.to(torch.bfloat16)
    tlo = (t - thi.float()).to(torch.bfloat16)
    u = K.gemm_bf16(W.up, thi, out_f32=True) + K.gemm_bf16(W.up, tlo, out_f32=True)
    call("gr_up_epilogue", "pppiii", ptr(u), ptr(normed), ptr(mixed), rows, H, hc)
    return mixed, post


def gr_mix(streams, W: GatedResidualWeights, eps, prev_post=None, prev_y=None):
    """The gated-residual read step: (mixed, post) of ``gr_mix_prenormed`` over ``gr_norm`` of the streams."""
    return gr_mix_prenormed(gr_norm(streams, W.norm, eps, prev_post, prev_y), W)


def shared_gate(x, w):
    """gate[r] = sigmoid(x[r] . w): the shared expert's scalar output gate."""
    if not x.is_cuda:
        return torch.sigmoid(x.float() @ w.float())
    g = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    call("gr_shared_gate", "pppii", ptr(x), ptr(w), ptr(g), x.shape[0], x.shape[1])
    return g


def stream_norm(streams, w, eps):
    """bf16 [rows * hc, H] of the per-stream RMSNorm * (1 + w)."""
    rows, hc, H = streams.shape
    if not streams.is_cuda:
        return gr_norm(streams.clone(), w, eps).to(torch.bfloat16).reshape(rows * hc, H)
    hi = torch.empty(rows * hc, H, dtype=torch.bfloat16, device=streams.device)
    call("gr_norm", "pppppppiiif", ptr(streams), ptr(w), 0, ptr(hi), 0, 0, 0, rows, H, hc, float(eps))
    return hi


# ---------------------------------------------------------------------------------------------- n-gram layer
def ple_gate_and_norm(key, value, streams, norm_key_w, norm_query_w, norm_conv_w, eps, gate_scale):
    """key [rows, hc*H] bf16, value [rows, H] bf16, streams fp32 [rows, hc, H] -> (gated fp32 [rows, hc, H], normed bf16
    [rows, hc*H]): gate = <rmsnorm_k(key_s), rmsnorm_q(stream_s)>, gated = sigmoid(signed_sqrt(gate * scale)) * value,
    normed = rmsnorm_c(gated)."""
    rows, hc, H = streams.shape
    if not streams.is_cuda:
        k = key.float().reshape(rows, hc, H)
        v = value.float()
        kn = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + norm_key_w.float())[None]
        qn = streams * torch.rsqrt(streams.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + norm_query_w.float())[None]
        g = (kn * qn).sum(-1) * gate_scale
        sg = torch.sigmoid(torch.sign(g) * torch.sqrt(g.abs().clamp(min=1e-6)))
        gated = sg[:, :, None] * v[:, None, :]
        ig = torch.rsqrt(sg.pow(2) * v.pow(2).mean(-1)[:, None] + eps)
        normed = gated * ig[:, :, None] * (1.0 + norm_conv_w.float())[None]
        return gated, normed.to(torch.bfloat16).reshape(rows, hc * H)
    gated = torch.empty(rows, hc, H, dtype=torch.float32, device=streams.device)
    normed = torch.empty(rows, hc * H, dtype=torch.bfloat16, device=streams.device)
    call("ple_gate", "ppppppppiiiff", ptr(key), ptr(value), ptr(streams), ptr(norm_key_w), ptr(norm_query_w), ptr(norm_conv_w),
         ptr(gated), ptr(normed), rows, H, hc, float(eps), float(gate_scale))
    return gated, normed


def ple_conv_apply(normed, conv_w, ring, slot, pos, gated, streams, dilation):
    """streams += gated + silu(causal dilated depthwise conv of normed), then the rows enter the slot rings.
    normed bf16 [rows, C], conv_w bf16 [C, 4], ring bf16 [slots, 16, C], slot / pos int32 [rows]."""
    rows, C = normed.shape
    flat = streams.reshape(rows, C)
    if not normed.is_cuda:
        nf, acc = normed.float(), torch.zeros(rows, C)
        for r in range(rows):
            sl, p = int(slot[r]), int(pos[r])
            if sl < 0:
                continue
            for j in range(4):
                k = (3 - j) * dilation
                sp = p - k
                if sp < 0:
                    continue
                rr = r - k
                if k == 0 or (rr >= 0 and int(slot[rr]) == sl and int(pos[rr]) == sp):
                    xv = nf[r if k == 0 else rr]
                else:
                    xv = ring[sl, sp % PLE_RING].float()
                acc[r] += conv_w[:, j].float() * xv
            flat[r] += gated.reshape(rows, C)[r] + acc[r] * torch.sigmoid(acc[r])
        for r in range(rows):
            if int(slot[r]) >= 0:
                ring[int(slot[r]), int(pos[r]) % PLE_RING] = normed[r]
        return streams
    call("ple_conv", "pppppppiii", ptr(normed), ptr(conv_w), ptr(ring), ptr(slot), ptr(pos), ptr(gated), ptr(streams), rows, C,
         dilation)
    call("ple_ring", "ppppii", ptr(normed), ptr(ring), ptr(slot), ptr(pos), rows, C)
    return streams
