"""``volta_ppl``: perplexity of token sequences through the engine's prefill path, and what calibration needs from
the same pass.

  volta_ppl --model DIR (--file TEXT | --tokens-file FILE.pt | --prompts DIR) [--seq 2048] [--tokens N] [--chunk 512]
      cross-entropy / perplexity over the sequences (every position after the first of a sequence is scored)
  --calibrate --hessian-dir D [--hessian-layers lo-hi] [--route-dump FILE] [--route-layers L,L] [--inputs-out FILE]
      the same pass with the capture taps on: x^T x of every projection input (one file per layer and site), the MoE
      blocks' routed rows, and the token sequences themselves as the training inputs of the end-to-end tuner
  --topk-out FILE [--topk 64]
      the teacher of this text: per position the K most likely tokens with their log-probabilities and the
      log-mass outside them ({"k", "ids": [S, K] per sequence, "logp": [S, K], "tail": [S]})
  --kl-teacher FILE
      KL(teacher || model) of this checkpoint against such a teacher (the K tokens plus one bucket for the rest)

Single rank (the vocabulary-parallel head of a tensor-parallel model would need its shards gathered).
Reference: tests/4_coherence/test_ppl.cpp as documented in docs/QUANTIZATION.md:99,112 (``--calibrate``, ``--prompts``,
``--topk-out``, ``--kl-teacher``) and docs/TESTS.md.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

import torch
import torch.nn.functional as F


def sequence_logits(engine, tokens: list[int], chunk: int = 512, slot: int = 0):
    """Yields (first position, fp32 logits [rows, vocab]) chunk by chunk for one sequence from position 0."""
    from ..runtime.batch import BatchRows, LOGITS_ALL
    model, kv = engine.model, engine.kv
    kv.reserve(slot, len(tokens) + 1)
    G = model.nq // model.nkv
    vocab = model.cfg.vocab
    for lo in range(0, len(tokens), chunk):
        ids = tokens[lo:lo + chunk]
        b = BatchRows.make(ids, list(range(lo, lo + len(ids))), [slot] * len(ids), engine.device, LOGITS_ALL, G, prefill=True)
        yield lo, model.forward(b, kv)[:, :vocab].float()


def topk_teacher(logits: torch.Tensor, k: int):
    """-> (ids [S, k] int32, logp [S, k] fp32, tail [S] fp32 = log of the probability mass outside the k tokens)."""
    lp = F.log_softmax(logits.float(), dim=-1)
    v, i = lp.topk(k, dim=-1)
    rest = (1.0 - v.exp().sum(-1)).clamp(min=1e-12)
    return i.int(), v, rest.log()


def kl_topk(student_logits: torch.Tensor, ids: torch.Tensor, logp: torch.Tensor, tail: torch.Tensor) -> torch.Tensor:
    """KL(teacher || student) per position over the teacher's K tokens and one bucket for everything else."""
    sl = F.log_softmax(student_logits.float(), dim=-1).gather(1, ids.long())
    s_rest = (1.0 - sl.exp().sum(-1)).clamp(min=1e-12).log()
    return (logp.exp() * (logp - sl)).sum(-1) + tail.exp() * (tail - s_rest)


def read_sequences(a, tokenizer) -> list[list[int]]:
    seqs: list[list[int]] = []
    if a.tokens_file:
        seqs = [[int(t) for t in s] for s in torch.load(a.tokens_file, weights_only=True)]
    elif a.prompts:
        for f in sorted(Path(a.prompts).glob("*.txt")):
            seqs.append(tokenizer.encode(f.read_text(errors="replace"))[: a.seq])
    else:
        ids = tokenizer.encode(Path(a.file).read_text(errors="replace"))
        if a.tokens:
            ids = ids[: a.tokens]
        seqs = [ids[i:i + a.seq] for i in range(0, len(ids), a.seq)]
    seqs = [s for s in seqs if len(s) >= 2]
    if a.tokens and not a.file:
        out, left = [], a.tokens
        for s in seqs:
            if left <= 0:
                break
            out.append(s[:left])
            left -= len(out[-1])
        seqs = [s for s in out if len(s) >= 2]
    return seqs


def run(engine, seqs, chunk: int = 512, topk: int = 0, teacher: dict | None = None, log=print) -> dict:
    """Scores the sequences one after another in slot 0. -> {"nll", "tokens", "ppl", "kl"?, "teacher"?}."""
    nll, count, kl_sum, kl_n = 0.0, 0, 0.0, 0
    out_t = {"k": topk, "ids": [], "logp": [], "tail": []} if topk else None
    for si, seq in enumerate(seqs):
        engine.kv.release(0)
        parts = []
        tgt = torch.tensor(seq[1:], dtype=torch.long, device=engine.device)
        for lo, lg in sequence_logits(engine, seq, chunk):
            hi = min(lo + lg.shape[0], len(seq) - 1)
            if hi > lo:
                nll += float(F.cross_entropy(lg[: hi - lo], tgt[lo:hi], reduction="sum"))
                count += hi - lo
            if teacher is not None:
                t_ids = teacher["ids"][si][lo:lo + lg.shape[0]].to(engine.device)
                t_lp = teacher["logp"][si][lo:lo + lg.shape[0]].to(engine.device)
                t_tail = teacher["tail"][si][lo:lo + lg.shape[0]].to(engine.device)
                kl = kl_topk(lg[: t_ids.shape[0]], t_ids, t_lp, t_tail)
                kl_sum += float(kl.sum())
                kl_n += kl.numel()
            if out_t is not None:
                parts.append(tuple(x.cpu() for x in topk_teacher(lg, topk)))
        if out_t is not None:
            for key, j in (("ids", 0), ("logp", 1), ("tail", 2)):
                out_t[key].append(torch.cat([p[j] for p in parts]))
        log(f"sequence {si}: {len(seq)} tokens, running ppl {math.exp(nll / max(count, 1)):.4f}")
    res = {"nll": nll / max(count, 1), "tokens": count, "ppl": math.exp(nll / max(count, 1))}
    if teacher is not None:
        res["kl"] = kl_sum / max(kl_n, 1)
    if out_t is not None:
        res["teacher"] = out_t
    return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="volta_ppl", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--file", default="")
    ap.add_argument("--tokens-file", default="", help="torch file: list of int token tensors")
    ap.add_argument("--prompts", default="", help="directory of *.txt, one sequence each")
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=0)
    ap.add_argument("--chunk", type=int, default=512)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--kv-format", default="bf16")
    ap.add_argument("--calibrate", action="store_true")
    ap.add_argument("--hessian-dir", default="")
    ap.add_argument("--hessian-layers", default="")
    ap.add_argument("--route-dump", default="")
    ap.add_argument("--route-layers", default="")
    ap.add_argument("--route-max-rows", type=int, default=8192)
    ap.add_argument("--inputs-out", default="")
    ap.add_argument("--topk-out", default="")
    ap.add_argument("--topk", type=int, default=64)
    ap.add_argument("--kl-teacher", default="")
    a = ap.parse_args(argv)
    if sum(bool(x) for x in (a.file, a.tokens_file, a.prompts)) != 1:
        ap.error("give exactly one of --file, --tokens-file, --prompts")
    from ..models.factory import load_model
    from ..ops.hessian import parse_layer_range
    from ..runtime.engine import Engine
    from ..runtime.kv_cache import PagedKVCache
    from ..runtime.route_dump import RouteRecorder
    model, _ = load_model(a.model, a.device)
    tok = None
    if not a.tokens_file:
        from ..loader.tokenizer import Tokenizer
        tok = Tokenizer.load(a.model)
    seqs = read_sequences(a, tok)
    if not seqs:
        print("volta_ppl: no sequence of two tokens or more", file=sys.stderr)
        return 1
    longest = max(len(s) for s in seqs)
    cfg = model.cfg
    kv = PagedKVCache(getattr(model, "kv_layers", cfg.n_layers), model.nkv, cfg.head_dim, (longest + 64) // 64 + 2, 1,
                      longest + 64, a.device, dtype=a.kv_format)
    engine = Engine(model, kv, use_graphs=False, prefill_chunk=a.chunk)
    hs = rec = None
    if a.calibrate:
        if a.hessian_dir:
            if not hasattr(model, "enable_hessians"):
                ap.error("this model family has no capture taps")
            hs = model.enable_hessians(parse_layer_range(a.hessian_layers, cfg.n_layers))
        if a.route_dump:
            layers = [int(x) for x in a.route_layers.split(",") if x] or None
            rec = model.route_recorder = RouteRecorder(layers, a.route_max_rows)
    teacher = torch.load(a.kl_teacher, weights_only=True) if a.kl_teacher else None
    with torch.no_grad():
        res = run(engine, seqs, a.chunk, a.topk if a.topk_out else 0, teacher)
    if hs is not None:
        files = hs.dump(a.hessian_dir)
        print(f"volta_ppl: {len(files)} capture files written to {a.hessian_dir}")
    if rec is not None:
        rec.save(a.route_dump)
    if a.inputs_out:
        torch.save([torch.tensor(s, dtype=torch.int32) for s in seqs], a.inputs_out)
    if a.topk_out:
        torch.save(res.pop("teacher"), a.topk_out)
    print(json.dumps({k: v for k, v in res.items() if k != "teacher"}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
