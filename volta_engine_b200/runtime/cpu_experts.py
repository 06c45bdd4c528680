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

from .._lib import call, ptr
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


class CpuExpertService:
    def __init__(self, threads: int = 4, spin_us: int = 200):
        self.experts: dict = {}          # (layer, expert id) -> HostExpert
        self.mailboxes: list = []
        self.seen: list = []
        self.threads, self.spin_us = threads, spin_us
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
        for r in range(n):                              # route order: deterministic sums
            row, e = int(mb.routes[r, 0]), int(mb.routes[r, 1])
            he = self.experts.get((layer, e))
            if he is None:
                mb.hdr[6] = 1
                continue
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


def attach_cpu_experts(model, host_fraction: float, service: CpuExpertService | None = None, budget_ms: float = 2000.0):
    """Move the last ``host_fraction`` of every MoE layer's experts to the host service (their device weights are zeroed,
    which makes an unnoticed route to them visible). Returns the service (started)."""
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
            gu = qn.dequantize_nvfp4(bank.gu_p[e].cpu(), bank.gu_s[e].cpu(), float(bank.gu_g[e]))
            dn = qn.dequantize_nvfp4(bank.dn_p[e].cpu(), bank.dn_s[e].cpu(), float(bank.dn_g[e]))
            service.add_expert(li, bank.e0 + e, HostExpert(gu, dn, 0 if cfg.act == "silu" else 1, cfg.act_limit))
            bank.gu_p[e].zero_()
            bank.dn_p[e].zero_()
        L.cpu = CpuExpertLayer(service, mb, li, owner.to(model.device), budget_ms)
    return service.start()
