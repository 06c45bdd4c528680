"""EXL3 (trellis-coded) weight format in vectorised PyTorch: decode oracle, Hadamard rotations, the linear
definition, a Viterbi encoder for small matrices and a synthetic random-code generator.

Format (reference statement: src/kernels/slang/ref_trellis.slang:1-15,37-69 and
src/backend/cpu/linear_trellis.cpp:69-78,129-180): ``codes`` uint16 ``[K/16, N/16, 16*bits]``; each 16x16 tile
holds 256 codes of ``bits`` bits as one cyclic bit stream (uint16 pairs form little-endian 32-bit words that are
read MSB first). Position p owns the 16-bit window starting at stream bit ``(p*bits + bits - 16) mod 256*bits``;
the window goes through a multiply-and-mask codebook to one fp16 value. Position p = 8*L + i sits at
``row = (L&3)*2 + (i&1) + 8*((i>>1)&1)``, ``col = 2*(L//8 + 4*(i>>2)) + ((L>>2)&1)`` of the tile.
``Linear(x) = had128(had128(x * suh) @ W) * svh`` with the normalised 128-point Walsh-Hadamard transform.
Codebooks: 0 = 3INST, 1 = MCG, 2 = MUL1.
"""
from __future__ import annotations

import math

import torch

CB_3INST, CB_MCG, CB_MUL1 = 0, 1, 2
_H_A = float(torch.tensor(0x1EEE, dtype=torch.int16).view(torch.float16))     # MUL1 slope
_H_B = float(torch.tensor(0xC931 - 65536, dtype=torch.int16).view(torch.float16))   # MUL1 offset


def _half_bits(u: torch.Tensor) -> torch.Tensor:
    """uint16 patterns held in int64 -> float32 values of those fp16 numbers."""
    u = u & 0xFFFF
    s = torch.where(u >= 32768, u - 65536, u).to(torch.int16)
    return s.view(torch.float16).float()


def decode_windows(w: torch.Tensor, cb: int = CB_MUL1) -> torch.Tensor:
    """16-bit windows (int64 tensor) -> fp32 values rounded to fp16 like the reference kernels."""
    w = w.to(torch.int64) & 0xFFFF
    if cb == CB_MUL1:
        x = (w * 0x83DCD12D) & 0xFFFFFFFF
        s = (x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + (x >> 24)
        v = (1024 + s).float() * _H_A + _H_B
        return v.to(torch.float16).float()
    x = ((w * 89226354 + 64248484) if cb == CB_3INST else (w * 0xCBAC1FED)) & 0xFFFFFFFF
    y = (x & 0x8FFF8FFF) ^ 0x3B603B60
    return (_half_bits(y & 0xFFFF) + _half_bits(y >> 16)).to(torch.float16).float()


def _tile_positions(layout: str = "stock"):
    """(row, col) inside the 16x16 tile of every stream position. "stock" is the exllamav3 order (mma.m16n8k16
    fragments); "volta" is the reference engine's own order (one column and eight consecutive rows per lane)."""
    p = torch.arange(256)
    L, i = p // 8, p % 8
    if layout == "volta":
        row = (i & 3) + 4 * (i >> 2) + 8 * ((L >> 3) & 1)
        col = (L & 3) + 4 * ((L >> 4) & 1) + 8 * ((L >> 2) & 1)
        return row, col
    row = (L & 3) * 2 + (i & 1) + 8 * ((i >> 1) & 1)
    col = 2 * (L // 8 + 4 * (i >> 2)) + ((L >> 2) & 1)
    return row, col


def is_half_rate(codes: torch.Tensor) -> bool:
    """A tile of 16 K + 8 code words holds the half-integer rate K + 0.5."""
    return codes.shape[-1] % 16 == 8


def tile_windows(codes: torch.Tensor, bits: int, tstart: torch.Tensor | None = None) -> torch.Tensor:
    """codes uint16/int [..., 16*bits] -> windows int64 [..., 256] in position order.

    ``tstart`` [...] (uint16 per tile, the extended trellis): the tile was encoded without the tail-biting ring, and the
    bits in front of its stream are the low bits of its start state instead of the tile's last bits; a window that ends
    before bit 16 takes its leading bits from there (the state's bit 0 sits directly in front of the stream).

    Half-integer rates (last dim 16 * bits + 8, the rate bits + 0.5): the windows of a tile advance by ``bits`` and
    ``bits + 1`` bits alternately, so position 2 j ends at bit j (2 bits + 1) + bits and position 2 j + 1 at
    (j + 1) (2 bits + 1); the stream is cyclic over the tile like the integer rates'."""
    c = codes.to(torch.int64) & 0xFFFF
    half = c.shape[-1] == 16 * bits + 8
    assert half or c.shape[-1] == 16 * bits, f"{c.shape[-1]} code words per tile do not hold {bits} (or {bits}.5) bits per weight"
    nw = c.shape[-1] // 2                                       # 32-bit words per tile
    words = c[..., 0::2] | (c[..., 1::2] << 16)                 # little-endian pairs
    total = nw * 32
    # expand the stream to bits (MSB first inside a word), cyclic
    shifts = torch.arange(31, -1, -1, device=c.device)
    stream = ((words[..., :, None] >> shifts) & 1).reshape(*c.shape[:-1], total)
    p = torch.arange(256, device=c.device)
    end = ((p // 2) * (2 * bits + 1) + torch.where(p % 2 == 0, bits, 2 * bits + 1)) if half else (p + 1) * bits
    start = (end - 16) % total
    idx = (start[:, None] + torch.arange(16, device=c.device)[None, :]) % total          # [256, 16]
    win_bits = stream[..., idx]                                                           # [..., 256, 16]
    weights = (1 << torch.arange(15, -1, -1, device=c.device)).to(torch.int64)
    win = (win_bits * weights).sum(-1)
    if tstart is not None:
        assert not half, "the extended trellis is defined for integer rates"
        st = tstart.to(torch.int64) & 0xFFFF
        for pos in range(256):
            e = int(end[pos])
            if e >= 16:
                break
            head = (words[..., 0] >> (32 - e)) & ((1 << e) - 1)                          # the stream's first e bits
            win[..., pos] = ((st & ((1 << (16 - e)) - 1)) << e) | head
    return win


def tile_gain(code: torch.Tensor) -> torch.Tensor:
    """Gain of a tile from its 8-bit code: (896 + c) / 1024, i.e. 0.875 .. 1.124."""
    return (896.0 + (code.to(torch.int64) & 0xFF).float()) / 1024.0


def reconstruct(codes: torch.Tensor, bits: int, cb: int = CB_MUL1, layout: str = "stock", tstart: torch.Tensor | None = None,
                tgain: torch.Tensor | None = None) -> torch.Tensor:
    """codes [K/16, N/16, 16*bits] (or 16*bits + 8: the rate bits + 0.5) -> W fp32 [K, N] in the rotated basis (no suh /
    svh). ``tstart`` / ``tgain`` [K/16, N/16]: the extended trellis' per-tile start states and gain codes."""
    KT, NT = codes.shape[0], codes.shape[1]
    vals = decode_windows(tile_windows(codes, bits, tstart), cb)        # [KT, NT, 256]
    if tgain is not None:                                       # per-tile gain, the product rounded to fp16 like the values
        vals = (vals * tile_gain(tgain)[..., None]).to(torch.float16).float()
    row, col = _tile_positions(layout)
    tile = torch.zeros(KT, NT, 16, 16, dtype=torch.float32, device=codes.device)
    tile[:, :, row.to(codes.device), col.to(codes.device)] = vals
    return tile.permute(0, 2, 1, 3).reshape(KT * 16, NT * 16)


def had128(x: torch.Tensor) -> torch.Tensor:
    """Normalised Walsh-Hadamard transform over blocks of 128 along the last dim (natural order)."""
    shp = x.shape
    v = x.float().reshape(-1, shp[-1] // 128, 128)
    h = 1
    while h < 128:
        v = v.reshape(v.shape[0], v.shape[1], 128 // (2 * h), 2, h)
        a, b = v[..., 0, :], v[..., 1, :]
        v = torch.stack((a + b, a - b), dim=-2).reshape(v.shape[0], v.shape[1], 128)
        h *= 2
    return (v * (1.0 / math.sqrt(128.0))).reshape(shp)


def linear_reference(x: torch.Tensor, codes: torch.Tensor, bits: int, suh: torch.Tensor, svh: torch.Tensor,
                     cb: int = CB_MUL1, layout: str = "stock", tstart=None, tgain=None) -> torch.Tensor:
    """fp32 statement of the EXL3 linear: x [M, K] -> [M, N]."""
    W = reconstruct(codes, bits, cb, layout, tstart, tgain)
    t = had128(x.float() * suh.float())
    return had128(t @ W) * svh.float()


def effective_weight(codes, bits, suh, svh, cb=CB_MUL1, layout="stock", tstart=None, tgain=None) -> torch.Tensor:
    """Dense [K, N] matrix equal to the whole linear map (for tests): row k = Linear(e_k)."""
    K = codes.shape[0] * 16
    return linear_reference(torch.eye(K, device=codes.device), codes, bits, suh, svh, cb, layout, tstart, tgain)


# ------------------------------------------------------------------------------------------------ synthesis
def random_codes(K: int, N: int, bits: int, gen: torch.Generator | None = None, device="cpu") -> torch.Tensor:
    """Uniform random bit streams. Random windows decode to a near-Gaussian unit-variance codebook value, which is
    what a trellis encoding of random N(0, sigma) weights looks like once sigma sits in the suh / svh scales."""
    words = int(16 * bits)                                    # bits may be K + 0.5: 16 K + 8 code words per tile
    return torch.randint(0, 65536, (K // 16, N // 16, words), generator=gen, device=device, dtype=torch.int32).to(torch.int16)


def synth_linear(K: int, N: int, bits: int, std: float = 0.02, gen=None, device="cpu"):
    """-> (codes int16, suh fp16 [K], svh fp16 [N]) of a random EXL3 linear whose effective weights have ~std."""
    codes = random_codes(K, N, bits, gen, device)
    sg = torch.randint(0, 2, (K,), generator=gen, device=device).float() * 2 - 1
    suh = sg.to(torch.float16)
    sv = (torch.randint(0, 2, (N,), generator=gen, device=device).float() * 2 - 1) * std
    return codes, suh, sv.to(torch.float16)


# ------------------------------------------------------------------------------------------------ encoder
def viterbi_encode_tile(target: torch.Tensor, bits: int, cb: int = CB_MUL1) -> torch.Tensor:
    """Trellis-encode one tile: ``target`` [256] values in position order -> uint16 code words [16*bits].

    Exact Viterbi over the 2^16-state bit-shift trellis (state = current 16-bit window), made tail-biting by
    two passes: the first pass runs an open trellis, the second starts from the state that ended the first and
    is forced to return to it. Cost O(256 * 2^16 * 2^bits); meant for the quantisation tool and tests.
    """
    dev = target.device
    S, B = 65536, 1 << bits
    vals = decode_windows(torch.arange(S, device=dev), cb)                 # value of every state
    states = torch.arange(S, device=dev)
    preds = (states[:, None] >> bits) | (torch.arange(B, device=dev)[None, :] << (16 - bits))   # [S, B]

    def run(start_state: int | None):
        if start_state is None:
            cost = (vals - target[0]) ** 2
        else:
            # position 0's window must be consistent with the cyclic wrap: it shares 16-bits bits with the end
            cost = torch.full((S,), float("inf"), device=dev)
            hi = start_state & ((1 << (16 - bits)) - 1)                    # low bits of the final window
            cand = (hi << bits) | torch.arange(B, device=dev)
            cost[cand] = (vals[cand] - target[0]) ** 2
        back = torch.empty(255, S, dtype=torch.int16, device=dev)
        for p in range(1, 256):
            c = cost[preds]                                                # [S, B]
            best, arg = c.min(dim=1)
            back[p - 1] = arg.to(torch.int16)
            cost = best + (vals - target[p]) ** 2
        return cost, back

    cost, back = run(None)
    end = int(cost.argmin())
    cost2, back2 = run(end)
    end2 = end if torch.isfinite(cost2[end]) else int(cost2.argmin())
    path = [end2]
    s = end2
    for p in range(254, -1, -1):
        s = int(preds[s, int(back2[p, s])])
        path.append(s)
    path.reverse()                                                         # window of every position
    total = 256 * bits
    stream = torch.zeros(total, dtype=torch.int64)
    for p, w in enumerate(path):
        start = (p * bits + bits - 16) % total
        for j in range(16):
            stream[(start + j) % total] = (w >> (15 - j)) & 1
    words = (stream.reshape(-1, 32) * (1 << torch.arange(31, -1, -1))).sum(-1)
    out = torch.stack((words & 0xFFFF, words >> 16), dim=-1).reshape(-1)   # little-endian uint16 pairs
    return torch.where(out >= 32768, out - 65536, out).to(torch.int16)


def quantize(W: torch.Tensor, bits: int, cb: int = CB_MUL1, seed: int = 0):
    """Quantise a dense [K, N] weight (y = x @ W): random-sign Hadamard rotation of both sides, per-channel scales,
    Viterbi per tile. Returns (codes, suh, svh). O(tiles * 2^(16+bits) * 256): small matrices only."""
    K, N = W.shape
    assert K % 128 == 0 and N % 128 == 0
    g = torch.Generator().manual_seed(seed)
    su = (torch.randint(0, 2, (K,), generator=g).float() * 2 - 1).to(W.device)
    sv = (torch.randint(0, 2, (N,), generator=g).float() * 2 - 1).to(W.device)
    # x W = x Su H Wq H Sv  =>  Wq = H (Su W Sv) H   (H symmetric orthonormal, sign matrices self-inverse)
    Wr = had128((had128((W.float() * su[:, None] * sv[None, :]).t().contiguous())).t().contiguous())
    scale = Wr.std().clamp(min=1e-12)          # codebook values have ~unit variance
    Wn = Wr / scale
    row, col = _tile_positions()
    if W.is_cuda and 2 <= bits <= 8:
        # every tile at once on the device (csrc/cuda/exl3_quant.cu): [K/16, N/16, 256] targets in stream-position order
        from ..ops.linear_exl3 import exl3_viterbi
        tiles = Wn.reshape(K // 16, 16, N // 16, 16).permute(0, 2, 1, 3)[:, :, row.to(W.device), col.to(W.device)]
        codes = exl3_viterbi(tiles.reshape(-1, 256).float().contiguous(), bits, cb).reshape(K // 16, N // 16, 16 * bits)
        return codes, su.to(torch.float16), (sv * scale).to(torch.float16)
    codes = torch.zeros(K // 16, N // 16, 16 * bits, dtype=torch.int16)
    for kt in range(K // 16):
        for nt in range(N // 16):
            tile = Wn[kt * 16:(kt + 1) * 16, nt * 16:(nt + 1) * 16]
            codes[kt, nt] = viterbi_encode_tile(tile[row, col].contiguous(), bits, cb).cpu()
    return codes.to(W.device), su.to(torch.float16), (sv * scale).to(torch.float16)
