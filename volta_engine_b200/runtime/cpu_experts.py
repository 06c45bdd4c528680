"""CPU expert service: experts that live in host memory are evaluated by a host thread pool while the GPU runs the
device-resident experts of the same layer; the two halves meet through a mailbox in pinned mapped memory
(csrc/cuda/cpu_experts.cu).

One mailbox per rank. The dispatcher thread polls the request sequence number, evaluates the requested routes
(``weight * down(act(gate(x)) * up(x))`` per route, summed per row in route order, fp32) and publishes the result with the
same sequence number. The device side waits with a wall-clock budget and reports expiry through the status word, so a stopped
or slow service degrades into a recorded error, never a hang.
Reference: inc/engine/runtime/cpu_expert_service.h:13-60 (service, mailboxes, dispatcher), src/runtime/cpu_expert_*.cpp,
src/kernels/cpu/nvfp4_linear.cpp (host linears).
"""
from __future__ import annotations

import threading
import time

import numpy as np
import torch

import ctypes

from .._lib import call, hcall, ptr
from ..quant import nvfp4 as qn

MB_ROWS, MAX_ROUTES, OFF_ROUTES = 16, 512, 64
OFF_X = OFF_ROUTES + MAX_ROUTES * 16


class Mailbox:
    def __init__(self, hidden: int, device):
        self.hidden = hidden
        nbytes = OFF_X + MB_ROWS * hidden * 2 + MB_ROWS * hidden * 4
        cuda = torch.device(device).type == "cuda"
        self.buf = torch.zeros(nbytes, dtype=torch.uint8)
        if cuda:
            self.buf = self.buf.pin_memory()              # pinned memory is mapped into the device address space (UVA)
        self.np = self.buf.numpy()
        self.hdr = self.np[:64].view(np.int64)
        self.routes = self.np[OFF_ROUTES:OFF_X].view(np.int32).reshape(MAX_ROUTES, 4)
        self.route_w = self.np[OFF_ROUTES:OFF_X].view(np.float32).reshape(MAX_ROUTES, 4)
        self.x = self.buf[OFF_X:OFF_X + MB_ROWS * hidden * 2].view(torch.bfloat16).reshape(MB_ROWS, hidden)
        self.out = self.np[OFF_X + MB_ROWS * hidden * 2:].view(np.float32).reshape(MB_ROWS, hidden)
        self.ctl = torch.zeros(2, dtype=torch.int64, device=device)       # [0] sequence to wait for (0: none), [1] running


class HostExpert:
    """fp32 host copies of one expert's matrices (dequantised once when the expert is attached)."""

    def __init__(self, gate_up: torch.Tensor, down: torch.Tensor, act: int = 0, limit: float = 0.0):
        self.gu, self.dn, self.act, self.limit = gate_up.float().contiguous(), down.float().contiguous(), act, limit

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gu = (x @ self.gu.t()).to(torch.bfloat16).float()
        inter = gu.shape[-1] // 2
        g, u = gu[..., :inter], gu[..., inter:]
        if self.limit > 0:
            g, u = g.clamp(max=self.limit), u.clamp(-self.limit, self.limit)
        a = torch.nn.functional.silu(g) if self.act == 0 else torch.nn.functional.gelu(g, approximate="tanh")
        return ((a * u).to(torch.bfloat16).float() @ self.dn.t()).to(torch.bfloat16).float()


class HostExpertNVFP4:
    """One expert kept in its packed NVFP4 form in host memory (4.5 bits per weight) and evaluated by the native host
    kernels (csrc/host/cpu_experts.cpp: byte-shuffle decode, AVX2 + FMA dot products, rows split over the pool's pinned
    workers). Same rounding points as :class:`HostExpert`."""

    def __init__(self, gu_p, gu_s, gu_g: float, dn_p, dn_s, dn_g: float, act: int = 0, limit: float = 0.0):
        self.gu_p, self.gu_s, self.dn_p, self.dn_s = (t.contiguous().cpu() for t in (gu_p, gu_s, dn_p, dn_s))
        self.gu_g, self.dn_g, self.act, self.limit = float(gu_g), float(dn_g), act, limit
        self.inter, self.hidden = self.gu_p.shape[0] // 2, self.dn_p.shape[0]
        self.scratch = torch.empty(3 * self.inter, dtype=torch.float32)

    def add_to(self, pool, x: torch.Tensor, out: torch.Tensor, weight: float) -> None:
        """out [hidden] fp32 += weight * expert(x [hidden] fp32)."""
        rc = hcall("cpu_nvfp4_expert", "pppfppfppiiiffp", pool, self.gu_p.data_ptr(), self.gu_s.data_ptr(), self.gu_g,
                   self.dn_p.data_ptr(), self.dn_s.data_ptr(), self.dn_g, x.data_ptr(), out.data_ptr(), self.hidden, self.inter,
                   self.act, float(self.limit), float(weight), self.scratch.data_ptr())
        if rc:
            raise ValueError("cpu_nvfp4_expert: dimensions must be multiples of 16")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.zeros(x.shape[0], self.hidden, dtype=torch.float32)
        xf = x.float().contiguous()
        for r in range(x.shape[0]):
            self.add_to(None, xf[r], out[r], 1.0)
        return out


def numa_node_cpus(node: int) -> list[int]:
    """CPU ids of a NUMA node from sysfs (empty when the node or the file does not exist)."""
    try:
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            return parse_cpu_list(f.read().strip())
    except OSError:
        return []


def parse_cpu_list(text: str) -> list[int]:
    """"0-3,8,10-11" -> [0, 1, 2, 3, 8, 10, 11]."""
    out = []
    for part in (p.strip() for p in text.split(",") if p.strip()):
        a, _, b = part.partition("-")
        out += list(range(int(a), int(b or a) + 1))
    return out


class CpuExpertService:
    def __init__(self, threads: int = 4, spin_us: int = 200, cpus: list[int] | None = None):
        self.experts: dict = {}          # (layer, expert id) -> HostExpert | HostExpertNVFP4
        self.mailboxes: list = []
        self.seen: list = []
        self.threads, self.spin_us = threads, spin_us
        self.cpus = list(cpus or [])
        self.pool = None                 # native worker pool (created by start(), workers pinned to ``cpus`` round robin)
        self._stop = threading.Event()
        self._th = None
        self.served = 0
        self.busy_s = 0.0

    def mailbox(self, hidden: int, device) -> Mailbox:
        mb = Mailbox(hidden, device)
        self.mailboxes.append(mb)
        self.seen.append(0)
        return mb

    def add_expert(self, layer: int, expert: int, he: HostExpert) -> None:
        self.experts[(layer, expert)] = he

    def start(self) -> "CpuExpertService":
        if self._th is None:
            torch.set_num_threads(max(torch.get_num_threads(), self.threads))
            if self.pool is None and any(isinstance(e, HostExpertNVFP4) for e in self.experts.values()):
                arr = (ctypes.c_int * max(1, len(self.cpus)))(*self.cpus) if self.cpus else None
                self.pool = hcall("cpu_pool_create", "ipii", self.threads, ctypes.addressof(arr) if arr is not None else 0,
                                  len(self.cpus), int(self.spin_us), restype=ctypes.c_void_p)
            self._stop.clear()
            self._th = threading.Thread(target=self._loop, name="cpu-experts", daemon=True)
            self._th.start()
        return self

    def stop(self) -> None:
        """Must run before the device context goes away: the mailboxes are mapped memory the dispatcher still reads."""
        self._stop.set()
        if self._th is not None:
            self._th.join(timeout=5)
            self._th = None
        if self.pool is not None:
            hcall("cpu_pool_destroy", "p", self.pool, restype=None)
            self.pool = None

    def _loop(self):
        while not self._stop.is_set():
            idle = True
            for i, mb in enumerate(self.mailboxes):
                seq = int(mb.hdr[0])
                if seq > self.seen[i]:
                    t0 = time.time()
                    self.handle(mb)
                    mb.hdr[1] = seq                     # published after the result rows (program order on the host)
                    self.seen[i] = seq
                    self.served += 1
                    self.busy_s += time.time() - t0
                    idle = False
            if idle:
                time.sleep(self.spin_us * 1e-6)

    def handle(self, mb: Mailbox) -> None:
        layer, rows, n, hidden = (int(v) for v in mb.hdr[2:6])
        out = np.zeros((rows, hidden), dtype=np.float32)
        x = mb.x[:rows].float()
        xt = ot = None
        for r in range(n):                              # route order: deterministic sums
            row, e = int(mb.routes[r, 0]), int(mb.routes[r, 1])
            he = self.experts.get((layer, e))
            if he is None:
                mb.hdr[6] = 1
                continue
            if isinstance(he, HostExpertNVFP4):
                if xt is None:
                    xt, ot = x.contiguous(), torch.from_numpy(out)
                he.add_to(self.pool, xt[row], ot[row], float(mb.route_w[r, 2]))
            else:
                out[row] += float(mb.route_w[r, 2]) * he.forward(x[row:row + 1])[0].numpy()
        mb.out[:rows] = out


class CpuExpertLayer:
    """Device-side handle of one MoE layer's host-owned experts."""

    def __init__(self, service: CpuExpertService, mailbox: Mailbox, layer: int, owner: torch.Tensor, budget_ms: float = 2000.0):
        self.service, self.mb, self.layer, self.owner = service, mailbox, layer, owner       # owner uint8 [e_local] on the device
        self.budget_ns = int(budget_ms * 1e6)

    def post(self, x, ids, w, e0: int, e_local: int) -> None:
        rows, topk = ids.shape
        call("cpu_post", "plppiiiiipppi", ptr(x), x.stride(0), ptr(ids), ptr(w), rows, topk, x.shape[1], e0, e_local,
             ptr(self.owner), self.mb.buf.data_ptr(), ptr(self.mb.ctl), self.layer)

    def wait_add(self, y) -> None:
        from ..ops.kernels import status_word
        call("cpu_wait_add", "pliipplp", ptr(y), y.stride(0), y.shape[0], y.shape[1], self.mb.buf.data_ptr(), ptr(self.mb.ctl),
             self.budget_ns, ptr(status_word(y.device)))


def attach_cpu_experts(model, host_fraction: float, service: CpuExpertService | None = None, budget_ms: float = 2000.0,
                       native: bool = True):
    """Move the last ``host_fraction`` of every MoE layer's experts to the host service (their device weights are zeroed,
    which makes an unnoticed route to them visible). ``native``: the experts stay packed and run on the native host
    kernels; otherwise fp32 copies evaluated with torch. Returns the service (started)."""
    service = service or CpuExpertService()
    cfg = model.cfg
    mb = service.mailbox(cfg.hidden, model.device)
    for li, L in enumerate(model.layers):
        bank = getattr(L, "bank", None)
        if bank is None or L.dense_ffn:
            continue
        E = bank.e_local
        n_host = int(E * host_fraction)
        owner = torch.zeros(E, dtype=torch.uint8)
        for e in range(E - n_host, E):
            owner[e] = 1
            act = 0 if cfg.act == "silu" else 1
            if native and bank.gu_p[e].shape[1] % 8 == 0 and bank.dn_p[e].shape[1] % 8 == 0:
                he = HostExpertNVFP4(bank.gu_p[e].cpu().clone(), bank.gu_s[e].cpu().clone(), float(bank.gu_g[e]),
                                     bank.dn_p[e].cpu().clone(), bank.dn_s[e].cpu().clone(), float(bank.dn_g[e]), act, cfg.act_limit)
            else:
                gu = qn.dequantize_nvfp4(bank.gu_p[e].cpu(), bank.gu_s[e].cpu(), float(bank.gu_g[e]))
                dn = qn.dequantize_nvfp4(bank.dn_p[e].cpu(), bank.dn_s[e].cpu(), float(bank.dn_g[e]))
                he = HostExpert(gu, dn, act, cfg.act_limit)
            service.add_expert(li, bank.e0 + e, he)
            bank.gu_p[e].zero_()
            bank.dn_p[e].zero_()
        L.cpu = CpuExpertLayer(service, mb, li, owner.to(model.device), budget_ms)
    return service.start()
