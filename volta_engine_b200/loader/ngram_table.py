"""Hashed n-gram embedding table (host side of the n-gram embedding layer): hash parameters, row ids of a position and
row decoding for the three storage forms. The table stays memory-mapped (tens of GB); a lookup touches a handful of rows
per token, so decoding happens on the host and only the gathered [rows, heads * 160] block goes to the GPU.

Storage forms (reference: inc/engine/loader/ngram_table.h:11-27, src/loader/ngram_table.cpp):
  trellis  one safetensors file; `*.shard_N.trellis` (or one `*.trellis`) uint16 [rows, 1 + 160*K/16]: word 0 an fp16 row
           scale, the rest a tail-biting bit ring; value i reads the 16-bit state whose bit m sits at ring bit
           ((i - m // K) mod 160) * K + m % K, decodes it with the MUL1 codebook, times the scale, plus the head's bias row.
  fp8      `<prefix>.ngram_embedding.shard_N.weight` uint8 E4M3 [rows, 160] and a bf16 `weight_scale`; no bias.
  gguf     one block-quantised tensor of every row (IQ4_NL, Q8_0, F16, BF16, F32) with the hash parameters in the file's
           metadata (`<arch>.ple.*`).
Hashing (ngram_table.cpp row_ids): for n = 2 .. ngram_size, mixed = tok[0]*mult[0] ^ tok[1]*mult[1] ^ ... ^ tok[n-1]*mult[n-1]
in wrapping int64 arithmetic; head h of that n-gram order reads row (mixed mod size[h]) + offset[h] (non-negative remainder).
"""
from __future__ import annotations

import numpy as np
import torch

from ..quant import exl3 as qx
from ..quant import gguf as gq
from ..quant import nvfp4 as qn
from .safetensors import SafeTensorsRepo

ROW_DIM = 160


def _wrap64(a: np.ndarray) -> np.ndarray:
    return a.astype(np.uint64).astype(np.int64)


class NgramTable:
    def __init__(self, head_offsets, head_sizes, multipliers, heads_per_ngram=None):
        self.head_offsets = np.asarray(head_offsets, dtype=np.int64)
        self.head_sizes = np.asarray(head_sizes, dtype=np.int64)
        self.multipliers = np.asarray(multipliers, dtype=np.int64)
        self.num_heads = len(self.head_offsets)
        self.ngram_size = len(self.multipliers)
        self.heads_per_ngram = heads_per_ngram or self.num_heads // (self.ngram_size - 1)
        assert self.num_heads == (self.ngram_size - 1) * self.heads_per_ngram and len(self.head_sizes) == self.num_heads
        self.kind = None
        self.rows_per_shard = 0
        self.shards: list = []
        self.head_bias = np.zeros((self.num_heads, ROW_DIM), dtype=np.float32)
        self.K = 6
        self.fp8_scale = 1.0
        self.gguf_type = 0
        self._codebook = None

    # ---- opening ---------------------------------------------------------------------------------------------------
    @classmethod
    def open_trellis(cls, path) -> "NgramTable":
        repo = SafeTensorsRepo(path) if not isinstance(path, SafeTensorsRepo) else path

        def find(suffix):
            hits = [n for n in repo.names() if n.endswith(suffix)]
            return hits[0] if hits else None
        t = cls(repo.load(find(".head_offsets")).numpy(), repo.load(find(".head_vocab_sizes")).numpy(),
                repo.load(find(".layer_multipliers")).numpy())
        t.K = int(repo.shards[0].metadata.get("K", "6"))
        t.head_bias = repo.load(find(".head_bias")).float().numpy().reshape(t.num_heads, ROW_DIM)
        s = 0
        while find(f".shard_{s}.trellis") is not None:
            t.shards.append(repo.load(find(f".shard_{s}.trellis")).numpy().view(np.uint16))
            s += 1
        if not t.shards and find(".trellis") is not None:
            t.shards.append(repo.load(find(".trellis")).numpy().view(np.uint16))
        assert t.shards, "n-gram table: no trellis shards"
        t.rows_per_shard = t.shards[0].shape[0]
        assert t.shards[0].shape[1] == 1 + ROW_DIM * t.K // 16
        t.kind = "trellis"
        t._codebook = qx.decode_windows(torch.arange(65536), qx.CB_MUL1).numpy()
        return t

    @classmethod
    def open_fp8(cls, repo: SafeTensorsRepo, prefix: str) -> "NgramTable":
        t = cls(repo.load(prefix + ".ngram_heads_offsets").numpy(), repo.load(prefix + ".ngram_heads_vocab_sizes").numpy(),
                repo.load(prefix + ".layer_multipliers").numpy())
        if repo.has(prefix + ".ngram_embedding.weight_scale"):
            t.fp8_scale = float(repo.load(prefix + ".ngram_embedding.weight_scale").float().reshape(-1)[0])
        s = 0
        while repo.has(f"{prefix}.ngram_embedding.shard_{s}.weight"):
            w = repo.load(f"{prefix}.ngram_embedding.shard_{s}.weight")
            assert w.ndim == 2 and w.shape[1] == ROW_DIM
            t.shards.append(w.view(torch.uint8).numpy())
            s += 1
        assert t.shards, "n-gram table: no FP8 shards"
        t.rows_per_shard = t.shards[0].shape[0]
        t.kind = "fp8"
        t._codebook = qn.e4m3_decode(torch.arange(256, dtype=torch.uint8)).float().numpy()
        return t

    @classmethod
    def open_gguf(cls, gguf, name: str) -> "NgramTable":
        arch = gguf.metadata["general.architecture"]
        md = gguf.metadata
        t = cls(md[f"{arch}.ple.head_offsets"], md[f"{arch}.ple.head_vocab_sizes"], md[f"{arch}.ple.layer_multipliers"],
                int(md[f"{arch}.ple.heads_per_ngram"]))
        assert int(md[f"{arch}.ple.ngram_size"]) == t.ngram_size
        info = gguf.tensors[name]
        assert info.shape[-1] == ROW_DIM
        if info.ggml_type not in (gq.GGML_IQ4_NL, gq.GGML_Q8_0, gq.GGML_F16, gq.GGML_BF16, gq.GGML_F32):
            raise ValueError(f"n-gram table: GGUF type {gq.NAMES.get(info.ggml_type, info.ggml_type)} is not read")
        raw = gguf.load(name)
        t.gguf_type = info.ggml_type
        t.shards = [raw.reshape(info.shape[0], -1) if raw.dtype == torch.uint8 else raw]
        t.rows_per_shard = info.shape[0]
        t.kind = "gguf"
        return t

    # ---- lookups ---------------------------------------------------------------------------------------------------
    def row_ids(self, tokens) -> np.ndarray:
        """tokens[0] is the token at the position, tokens[s] the one s positions earlier (the caller substitutes the eos id
        across segment boundaries). Returns the global row id of every head."""
        tok = np.asarray(tokens, dtype=np.int64)
        out = np.zeros(self.num_heads, dtype=np.int64)
        with np.errstate(over="ignore"):
            prods = _wrap64(tok[: self.ngram_size].astype(np.uint64) * self.multipliers.astype(np.uint64))
        for n in range(2, self.ngram_size + 1):
            mixed = np.int64(prods[0])
            for s in range(1, n):
                mixed = np.int64(mixed ^ prods[s])
            lo = (n - 2) * self.heads_per_ngram
            for h in range(lo, lo + self.heads_per_ngram):
                out[h] = int(mixed) % int(self.head_sizes[h]) + int(self.head_offsets[h])     # Python %: non-negative
        return out

    def decode_row(self, uid: int, head: int) -> np.ndarray:
        shard, local = divmod(int(uid), self.rows_per_shard)
        if self.kind == "gguf":
            row = self.shards[0][local]
            if self.gguf_type in gq.BLOCK and gq.BLOCK[self.gguf_type][0] > 1:
                return gq.dequantize(torch.as_tensor(row)[None], self.gguf_type, ROW_DIM)[0].numpy()
            return torch.as_tensor(row).float().numpy()
        if self.kind == "fp8":
            return self._codebook[self.shards[shard][local]] * np.float32(self.fp8_scale)
        row = self.shards[shard][local]
        scale = row[:1].view(np.float16).astype(np.float32)[0]
        bits = np.unpackbits(row[1:].view(np.uint8), bitorder="little")        # ring bit idx -> word idx>>4, bit idx&15
        K = self.K
        i = np.arange(ROW_DIM)[:, None]
        m = np.arange(16)[None, :]
        idx = ((i - m // K) % ROW_DIM) * K + m % K
        state = (bits[idx].astype(np.int64) << m).sum(1)
        return self._codebook[state] * scale + self.head_bias[head]

    def lookup(self, tokens) -> np.ndarray:
        """[num_heads * 160] fp32: the decoded rows of every head for one position, concatenated."""
        ids = self.row_ids(tokens)
        return np.concatenate([self.decode_row(ids[h], h) for h in range(self.num_heads)])

    def lookup_sequence(self, ids, eos_id: int = -1) -> torch.Tensor:
        """[len(ids), num_heads * 160] for a token sequence; history does not cross an eos token."""
        out = np.zeros((len(ids), self.num_heads * ROW_DIM), dtype=np.float32)
        for p in range(len(ids)):
            toks, cut = [], False
            for s in range(self.ngram_size):
                q = p - s
                if q < 0 or cut:
                    toks.append(eos_id if eos_id >= 0 else 0)
                    continue
                toks.append(int(ids[q]))
                if s > 0 and int(ids[q]) == eos_id:
                    cut = True
            out[p] = self.lookup(toks)
        return torch.from_numpy(out)


def encode_trellis_row(values: np.ndarray, K: int, codebook: np.ndarray, rng: np.random.Generator):
    """Test / tooling helper: a random valid ring (any bit ring decodes to codebook values) -> (row words, decoded values
    without scale and bias). ``values`` only fixes the length; the ring is drawn at random."""
    nbits = ROW_DIM * K
    bits = rng.integers(0, 2, nbits, dtype=np.uint8)
    words = np.packbits(bits, bitorder="little").view(np.uint16)
    i = np.arange(ROW_DIM)[:, None]
    m = np.arange(16)[None, :]
    idx = ((i - m // K) % ROW_DIM) * K + m % K
    state = (bits[idx].astype(np.int64) << m).sum(1)
    return words, codebook[state]
