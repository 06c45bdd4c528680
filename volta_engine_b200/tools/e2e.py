"""``volta_e2e``: end-to-end scale tuning of a quantised dense decoder against a teacher.

Every quantised linear is a frozen core between a per-input-channel and a per-output-channel scale
(``W = diag(su) T diag(sv)``; for EXL3 the core is the Hadamard-rotated trellis decode). The tool trains log deltas on all
those scales and additive deltas on the norm weights with Adam on KL(teacher || model) over token sequences; codes and
every other weight stay frozen. The model runs in an fp32 training form written in PyTorch (autograd), each layer
recomputed from its saved input in the backward (activation checkpointing). Learning rate: linear warm-up, then a cosine
down to ``lr_min * lr``. ``devices``: the layers are split evenly over the devices as sequential stages with hand-offs
between them (``--tp 0`` form of the reference tool).
Reference: docs/QUANTIZATION.md:99 (``volta_e2e``), src/tools/volta_e2e.cpp:473-512 (stage split), inc/engine/train/qwen4_exp.h.
"""
from __future__ import annotations

import argparse
import math
import sys
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint


class TunedLinear(torch.nn.Module):
    """y = ((x * su * exp(a_u)) @ T) * sv * exp(a_v) with T, su, sv frozen and the log deltas trained."""

    def __init__(self, core: torch.Tensor, su: torch.Tensor, sv: torch.Tensor):
        super().__init__()
        self.register_buffer("core", core.float().contiguous())          # [in, out]
        self.register_buffer("su", su.float().clone())
        self.register_buffer("sv", sv.float().clone())
        self.a_u = torch.nn.Parameter(torch.zeros_like(self.su))
        self.a_v = torch.nn.Parameter(torch.zeros_like(self.sv))

    @classmethod
    def from_exl3(cls, lin) -> "TunedLinear":
        from ..quant import exl3 as ex
        W = ex.reconstruct(lin.codes.cpu(), lin.bits, lin.cb, lin.layout)
        core = ex.had128(ex.had128(W.t()).t())
        return cls(core, lin.suh.cpu(), lin.svh.cpu())

    @classmethod
    def from_dense(cls, w: torch.Tensor) -> "TunedLinear":
        """[out, in] dense weight as a core with unit scales (formats without per-channel scales)."""
        return cls(w.float().t().contiguous(), torch.ones(w.shape[1]), torch.ones(w.shape[0]))

    def forward(self, x):
        return ((x * (self.su * torch.exp(self.a_u))) @ self.core) * (self.sv * torch.exp(self.a_v))

    def tuned_scales(self):
        return (self.su * torch.exp(self.a_u)).detach(), (self.sv * torch.exp(self.a_v)).detach()


class TunedNorm(torch.nn.Module):
    def __init__(self, w: torch.Tensor, eps: float, bias: float = 0.0):
        super().__init__()
        self.register_buffer("w0", w.float().clone())
        self.delta = torch.nn.Parameter(torch.zeros_like(self.w0))
        self.eps, self.bias = eps, bias

    def forward(self, x):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * (self.w0 + self.delta + self.bias)


def _rope(x, pos, theta, rot):
    """x [T, heads, hd], NeoX pairs on the first ``rot`` dims."""
    half = rot // 2
    inv = torch.exp2(-math.log2(theta) * (2.0 * torch.arange(half, device=x.device, dtype=torch.float32) / rot))
    ang = pos.float()[:, None] * inv[None]
    cs, sn = ang.cos()[:, None], ang.sin()[:, None]
    a, b = x[..., :half], x[..., half:rot]
    return torch.cat([a * cs - b * sn, b * cs + a * sn, x[..., rot:]], dim=-1)


class TunedLayer(torch.nn.Module):
    def __init__(self, cfg, lin: dict, norms: dict):
        super().__init__()
        self.cfg = cfg
        self.qkv, self.o, self.gu, self.dn = (lin[k] for k in ("qkv", "o", "gate_up", "down"))
        self.n1, self.n2 = norms["attn"], norms["ffn"]

    def forward(self, h):
        c = self.cfg
        T = h.shape[0]
        hd, nq, nkv = c.head_dim, c.n_q, c.n_kv
        qkv = self.qkv(self.n1(h))
        pos = torch.arange(T, device=h.device)
        rot = c.rot_dim or hd
        q = _rope(qkv[:, : nq * hd].reshape(T, nq, hd), pos, c.rope_theta, rot)
        k = _rope(qkv[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd), pos, c.rope_theta, rot)
        v = qkv[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
        g = nq // nkv
        att = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.repeat_interleave(g, 1).transpose(0, 1)[None],
                                             v.repeat_interleave(g, 1).transpose(0, 1)[None], is_causal=True,
                                             scale=c.attn_scale or 1.0 / math.sqrt(hd))[0].transpose(0, 1).reshape(T, nq * hd)
        h = h + self.o(att)
        gu = self.gu(self.n2(h))
        inter = gu.shape[-1] // 2
        act = F.silu(gu[:, :inter]) if c.act == "silu" else F.gelu(gu[:, :inter], approximate="tanh")
        return h + self.dn(act * gu[:, inter:])


@dataclass
class E2EOptions:
    steps: int = 64
    batch: int = 4
    lr: float = 1e-3
    warmup: int = 2
    lr_min: float = 0.1
    eval_every: int = 16
    norms: bool = True
    devices: list = field(default_factory=lambda: ["cpu"])


# ---------------------------------------------------------------------------------------------- tensor parallel form
class ShardedTunedLinear(torch.nn.Module):
    """A ``TunedLinear`` cut for one rank. ``split = "col"``: this rank's output features (``cols``), the input scale
    deltas replicated (their gradient is summed over the ranks); ``split = "row"``: this rank's input features, the output
    scale deltas replicated and applied by the caller after the partial sums are reduced (``finish``)."""

    def __init__(self, full: TunedLinear, split: str, idx: torch.Tensor):
        super().__init__()
        self.split = split
        if split == "col":
            self.register_buffer("core", full.core[:, idx].contiguous())
            self.register_buffer("su", full.su.clone())
            self.register_buffer("sv", full.sv[idx].clone())
        else:
            self.register_buffer("core", full.core[idx].contiguous())
            self.register_buffer("su", full.su[idx].clone())
            self.register_buffer("sv", full.sv.clone())
        self.a_u = torch.nn.Parameter(torch.zeros_like(self.su))
        self.a_v = torch.nn.Parameter(torch.zeros_like(self.sv))

    def forward(self, x):
        y = (x * (self.su * torch.exp(self.a_u))) @ self.core
        return y * (self.sv * torch.exp(self.a_v)) if self.split == "col" else y

    def finish(self, y):
        """Row-parallel: the output scales, on the reduced rows."""
        return y * (self.sv * torch.exp(self.a_v))

    def replicated(self):
        return [self.a_u] if self.split == "col" else [self.a_v]


class TunedLayerSP(torch.nn.Module):
    """``TunedLayer`` in the sequence-parallel form: every rank owns ``T / ranks`` rows of the fp32 stream and the heads /
    hidden units ``rank :: ranks`` of the sub-layers. A sub-layer normalises its rows, all-gathers them, runs its
    column-parallel and row-parallel linears on its slice and reduce-scatters the partial sums back to rows
    (``parallel.sequence_parallel``; the collectives are each other's gradient).
    Reference: inc/engine/train/qwen4_exp.h:15-20, src/train/qwen4_exp.cpp:229-259."""

    def __init__(self, layer: "TunedLayer", rank: int, world: int, group=None):
        super().__init__()
        c = layer.cfg
        self.cfg, self.rank, self.world, self.group = c, rank, world, group
        hd, nq, nkv = c.head_dim, c.n_q, c.n_kv
        assert nq % world == 0 and nkv % world == 0, "heads must divide by the rank count"
        self.nq, self.nkv = nq // world, nkv // world
        ar = torch.arange
        q = ar(rank * self.nq * hd, (rank + 1) * self.nq * hd)
        k = nq * hd + ar(rank * self.nkv * hd, (rank + 1) * self.nkv * hd)
        v = (nq + nkv) * hd + ar(rank * self.nkv * hd, (rank + 1) * self.nkv * hd)
        self.qkv = ShardedTunedLinear(layer.qkv, "col", torch.cat([q, k, v]))
        self.o = ShardedTunedLinear(layer.o, "row", q)
        inter = layer.gu.core.shape[1] // 2
        assert inter % world == 0
        f = inter // world
        gcols = ar(rank * f, (rank + 1) * f)
        self.gu = ShardedTunedLinear(layer.gu, "col", torch.cat([gcols, inter + gcols]))
        self.dn = ShardedTunedLinear(layer.dn, "row", gcols)
        self.n1, self.n2 = layer.n1, layer.n2

    def replicated(self):
        return self.qkv.replicated() + self.o.replicated() + self.gu.replicated() + self.dn.replicated() + [self.n1.delta, self.n2.delta]

    def forward(self, h):
        from ..parallel.sequence_parallel import gather_rows, reduce_scatter_rows
        c = self.cfg
        hd, nq, nkv = c.head_dim, self.nq, self.nkv
        x = gather_rows(self.n1(h), self.group)                         # [T, H]
        T = x.shape[0]
        qkv = self.qkv(x)
        pos = torch.arange(T, device=h.device)
        rot = c.rot_dim or hd
        q = _rope(qkv[:, : nq * hd].reshape(T, nq, hd), pos, c.rope_theta, rot)
        k = _rope(qkv[:, nq * hd:(nq + nkv) * hd].reshape(T, nkv, hd), pos, c.rope_theta, rot)
        v = qkv[:, (nq + nkv) * hd:].reshape(T, nkv, hd)
        g = nq // nkv
        att = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.repeat_interleave(g, 1).transpose(0, 1)[None],
                                             v.repeat_interleave(g, 1).transpose(0, 1)[None], is_causal=True,
                                             scale=c.attn_scale or 1.0 / math.sqrt(hd))[0].transpose(0, 1).reshape(T, nq * hd)
        h = h + self.o.finish(reduce_scatter_rows(self.o(att), self.group))
        gu = self.gu(gather_rows(self.n2(h), self.group))
        inter = gu.shape[-1] // 2
        act = F.silu(gu[:, :inter]) if c.act == "silu" else F.gelu(gu[:, :inter], approximate="tanh")
        return h + self.dn.finish(reduce_scatter_rows(self.dn(act * gu[:, inter:]), self.group))


class TunedModelSP(torch.nn.Module):
    """``TunedModel`` over a process group: rows sharded from the embedding to the logits (every rank scores its own
    rows against the teacher; the loss is the sum over ranks). ``sync_grads`` sums the gradients of the parameters every
    rank holds in full; sharded parameters keep their local gradients."""

    def __init__(self, full: "TunedModel", rank: int, world: int, device="cpu", group=None):
        super().__init__()
        self.cfg, self.rank, self.world, self.group = full.cfg, rank, world, group
        self.layers = torch.nn.ModuleList([TunedLayerSP(L, rank, world, group) for L in full.layers])
        self.final_norm = full.final_norm
        self.register_buffer("embed", full.embed.clone())
        self.register_buffer("head", full.head.clone())
        self.devices = [device]
        self.to(device)

    def rows(self, T: int) -> slice:
        per = T // self.world
        assert per * self.world == T, "sequence length must be a multiple of the rank count"
        return slice(self.rank * per, (self.rank + 1) * per)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """-> logits of this rank's rows [T / ranks, vocab]."""
        mine = ids[self.rows(ids.shape[0])]
        h = self.embed[mine.to(self.embed.device).long()] * self.cfg.embed_scale
        for L in self.layers:
            h = checkpoint(L, h, use_reentrant=False) if self.training else L(h)
        return self.final_norm(h) @ self.head.t()

    def sync_grads(self) -> None:
        from ..parallel.sequence_parallel import sum_replicated_grads
        reps = [self.final_norm.delta]
        for L in self.layers:
            reps += L.replicated()
        sum_replicated_grads(reps, self.group)


class TunedModel(torch.nn.Module):
    """fp32 training form of a dense decoder whose linears are ``TunedLinear`` (stacked qkv / gate_up like the engine)."""

    def __init__(self, cfg, embed, layers, final_norm, head, devices):
        super().__init__()
        self.cfg = cfg
        self.layers = torch.nn.ModuleList(layers)
        self.final_norm, self.devices = final_norm, devices
        n = len(layers)
        self.stage = [min(len(devices) - 1, i * len(devices) // max(1, n)) for i in range(n)]      # even split, in order
        for i, L in enumerate(self.layers):
            L.to(devices[self.stage[i]])
        self.register_buffer("embed", embed.float().to(devices[0]))
        self.final_norm.to(devices[-1])
        self.register_buffer("head", head.float().to(devices[-1]))

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        h = self.embed[ids.to(self.devices[0]).long()] * self.cfg.embed_scale
        for i, L in enumerate(self.layers):
            h = h.to(self.devices[self.stage[i]])                      # stage hand-off
            h = checkpoint(L, h, use_reentrant=False) if self.training else L(h)
        return self.final_norm(h.to(self.devices[-1])) @ self.head.t()


def build_from_engine_model(model, devices=("cpu",)) -> TunedModel:
    """Training form of an engine ``DenseModel`` whose linears are EXL3 (tuned) or anything else (dense core, unit scales)."""
    from ..ops.linear_exl3 import LinearEXL3

    def tl(lin):
        if isinstance(lin, LinearEXL3):
            return TunedLinear.from_exl3(lin)
        w = lin.weight if hasattr(lin, "weight") else lin.dequant()
        return TunedLinear.from_dense(w.float().cpu())
    cfg = model.cfg
    layers = []
    for L in model.layers:
        gu = L.gate_up
        if getattr(gu, "gated", False):
            raise ValueError("interleaved gate/up weights are a decode layout; tune the checkpoint form")
        layers.append(TunedLayer(cfg, {"qkv": tl(L.qkv), "o": tl(L.o_proj), "gate_up": tl(gu), "down": tl(L.down)},
                                 {"attn": TunedNorm(L.attn_norm.cpu(), cfg.rms_eps, cfg.norm_bias),
                                  "ffn": TunedNorm(L.ffn_norm.cpu(), cfg.rms_eps, cfg.norm_bias)}))
    head = model.lm_head.weight if hasattr(model.lm_head, "weight") else model.lm_head.dequant()
    return TunedModel(cfg, model.embed.cpu(), layers, TunedNorm(model.final_norm.cpu(), cfg.rms_eps, cfg.norm_bias),
                      head.cpu()[: cfg.vocab], list(devices))


def kl_teacher(student_logits: torch.Tensor, teacher_logits) -> torch.Tensor:
    """mean over positions of KL(teacher || student). The teacher is a full logits tensor, or the top-K form that
    ``volta_ppl --topk-out`` writes: (ids [S, K], logp [S, K], tail [S])."""
    if isinstance(teacher_logits, (tuple, list)):
        from .ppl import kl_topk
        ids, logp, tail = (t.to(student_logits.device) for t in teacher_logits)
        return kl_topk(student_logits[: ids.shape[0]], ids, logp, tail).mean()
    t = F.log_softmax(teacher_logits.float(), dim=-1)
    s = F.log_softmax(student_logits.float(), dim=-1)
    return (t.exp() * (t - s)).sum(-1).mean()


def _to(teacher, device):
    return tuple(t.to(device) for t in teacher) if isinstance(teacher, (tuple, list)) else teacher.to(device)


def lr_at(step: int, o: E2EOptions) -> float:
    if step < o.warmup:
        return o.lr * (step + 1) / max(1, o.warmup)
    p = (step - o.warmup) / max(1, o.steps - o.warmup)
    return o.lr * (o.lr_min + (1 - o.lr_min) * 0.5 * (1 + math.cos(math.pi * min(1.0, p))))


def tune(model: TunedModel, sequences: list, teachers: list, o: E2EOptions, held_out: int = 1, log=print) -> dict:
    """sequences: list of id tensors; teachers: matching teacher logits [T, vocab]. The last ``held_out`` sequences only
    evaluate. Returns {"eval": [(step, kl)], "train": [kl per step]}."""
    params = [p for n, p in model.named_parameters() if o.norms or not n.endswith("delta")]
    opt = torch.optim.Adam(params, lr=o.lr)
    train = list(range(len(sequences) - held_out))
    hist = {"eval": [], "train": []}

    sp = isinstance(model, TunedModelSP)

    def teacher_of(i, T):
        t = _to(teachers[i], model.devices[-1])
        if not sp:
            return t
        r = model.rows(T)                                   # this rank scores its own rows
        return tuple(x[r] for x in t) if isinstance(t, (tuple, list)) else t[r]

    def over_ranks(x: float) -> float:
        if not sp or model.world == 1:
            return x
        import torch.distributed as dist
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, group=model.group)
        return float(t) / model.world

    def evaluate(step):
        model.eval()
        with torch.no_grad():
            kl = sum(float(kl_teacher(model(sequences[i]), teacher_of(i, sequences[i].shape[0])))
                     for i in range(len(sequences) - held_out, len(sequences))) / max(1, held_out)
        kl = over_ranks(kl)
        hist["eval"].append((step, kl))
        log(f"step {step}: held-out KL {kl:.6f}")
        return kl
    evaluate(0)
    scale = o.batch * (model.world if sp else 1)
    for step in range(o.steps):
        model.train()
        for g in opt.param_groups:
            g["lr"] = lr_at(step, o)
        opt.zero_grad(set_to_none=True)
        total = 0.0
        for b in range(o.batch):
            i = train[(step * o.batch + b) % len(train)]
            loss = kl_teacher(model(sequences[i]), teacher_of(i, sequences[i].shape[0])) / scale
            loss.backward()
            total += float(loss.detach())
        if sp:
            model.sync_grads()                              # parameters every rank holds in full: sum over the ranks
            total = over_ranks(total) * model.world
        opt.step()
        hist["train"].append(total)
        if (step + 1) % o.eval_every == 0 or step + 1 == o.steps:
            evaluate(step + 1)
    return hist


def gather_tuned_model(sp: "TunedModelSP"):
    """The tuned scales of every rank put back into whole vectors (what the tool writes): an object with the attributes
    ``main`` reads (``layers[i].qkv / o / gu / dn`` with ``tuned_scales()``, ``n1`` / ``n2``)."""
    import torch.distributed as dist

    class _Lin:
        def __init__(self, su, sv):
            self.su, self.sv = su, sv

        def tuned_scales(self):
            return self.su, self.sv

    def whole(lin: ShardedTunedLinear):
        su = (lin.su * torch.exp(lin.a_u)).detach().cpu()
        sv = (lin.sv * torch.exp(lin.a_v)).detach().cpu()
        part = sv if lin.split == "col" else su
        parts = [torch.empty_like(part) for _ in range(sp.world)]
        dist.all_gather(parts, part.contiguous(), group=sp.group)
        return parts, (su if lin.split == "col" else sv)

    class _Layer:
        pass
    layers = []
    for L in sp.layers:
        out = _Layer()
        c = sp.cfg
        hd = c.head_dim
        parts, su = whole(L.qkv)                                        # per rank [q | k | v] slices -> [Q | K | V]
        nq, nkv = L.nq * hd, L.nkv * hd
        sv = torch.cat([p[:nq] for p in parts] + [p[nq:nq + nkv] for p in parts] + [p[nq + nkv:] for p in parts])
        out.qkv = _Lin(su, sv)
        parts, sv = whole(L.o)
        out.o = _Lin(torch.cat(parts), sv)
        parts, su = whole(L.gu)
        f = parts[0].shape[0] // 2
        out.gu = _Lin(su, torch.cat([p[:f] for p in parts] + [p[f:] for p in parts]))
        parts, sv = whole(L.dn)
        out.dn = _Lin(torch.cat(parts), sv)
        out.n1, out.n2 = L.n1, L.n2
        layers.append(out)

    class _Model:
        pass
    m = _Model()
    m.layers = layers
    return m


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="volta_e2e", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="quantised model directory (EXL3 linears are tuned)")
    ap.add_argument("--inputs", required=True, help="torch file: list of int token tensors")
    ap.add_argument("--teacher", required=True, help="torch file: list of teacher logits, or a model directory to run")
    ap.add_argument("--out", required=True)
    ap.add_argument("--devices", default="cpu")
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--lr-min", type=float, default=0.1)
    ap.add_argument("--eval-every", type=int, default=16)
    ap.add_argument("--norms", type=int, default=1)
    ap.add_argument("--tp", type=int, default=0,
                    help="N > 0: sequence-parallel tensor parallelism over the N ranks this process was started with "
                         "(python -m torch.distributed.run --nproc-per-node N -m volta_engine_b200.tools.e2e ...); "
                         "0: the layers are split over --devices as sequential stages")
    a = ap.parse_args(argv)
    from pathlib import Path
    from ..loader.safetensors import write_safetensors
    from ..models.factory import load_model
    devices = [d if d.startswith(("cpu", "cuda")) else f"cuda:{d}" for d in a.devices.split(",")]
    model, _ = load_model(a.model, "cpu", None)
    tm = build_from_engine_model(model, devices)
    seqs = torch.load(a.inputs, weights_only=True)
    if Path(a.teacher).is_dir():
        tmodel, _ = load_model(a.teacher, "cpu", None)
        teacher = build_from_engine_model(tmodel, devices).eval()
        with torch.no_grad():
            teachers = [teacher(s).cpu() for s in seqs]
    else:
        teachers = torch.load(a.teacher, weights_only=True)
        if isinstance(teachers, dict):                   # the top-K teacher of volta_ppl
            teachers = list(zip(teachers["ids"], teachers["logp"], teachers["tail"]))
    o = E2EOptions(a.steps, a.batch, a.lr, a.warmup, a.lr_min, a.eval_every, bool(a.norms), devices)
    rank = 0
    if a.tp > 0:
        import os
        import torch.distributed as dist
        cuda = devices[0].startswith("cuda")
        dist.init_process_group("nccl" if cuda else "gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        if world != a.tp:
            raise SystemExit(f"--tp {a.tp} but the process group has {world} ranks")
        dev = f"cuda:{int(os.environ.get('LOCAL_RANK', rank))}" if cuda else "cpu"
        tm = TunedModelSP(tm, rank, world, dev)
        # sequences are cut to a multiple of the rank count (rows are sharded evenly)
        seqs = [sq[: sq.shape[0] // world * world] for sq in seqs]
        teachers = [tuple(x[: sq.shape[0]] for x in t) if isinstance(t, (tuple, list)) else t[: sq.shape[0]]
                    for t, sq in zip(teachers, seqs)]
    hist = tune(tm, seqs, teachers, o, log=print if rank == 0 else (lambda *_: None))
    if a.tp > 0:
        tm = gather_tuned_model(tm)
        if rank != 0:
            return 0
    out = Path(a.out) / ".partial"
    out.mkdir(parents=True, exist_ok=True)
    tensors = {}
    for li, L in enumerate(tm.layers):
        for name, lin in (("qkv", L.qkv), ("o_proj", L.o), ("gate_up", L.gu), ("down", L.dn)):
            su, sv = lin.tuned_scales()
            tensors[f"layers.{li}.{name}.suh"], tensors[f"layers.{li}.{name}.svh"] = su.half().cpu(), sv.half().cpu()
        tensors[f"layers.{li}.attn_norm.weight"] = (L.n1.w0 + L.n1.delta).detach().half().cpu()
        tensors[f"layers.{li}.ffn_norm.weight"] = (L.n2.w0 + L.n2.delta).detach().half().cpu()
    write_safetensors(out / "e2e_scales.safetensors", tensors)
    print(f"held-out KL {hist['eval'][0][1]:.6f} -> {hist['eval'][-1][1]:.6f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
