"""W4A4 linears for activations that live in host memory.

The reference has no such path: its ops take CUDA tensors and its callers copy whole activation
matrices before and after (e.g. `x.cuda()` ... `.cpu()`).  When inputs and outputs are host
buffers, the PCIe transfers dominate (a Wan-14B QKV projection of 32760 tokens moves 0.34 GB in
and 1.0 GB out for 1.6 ms of GEMM), so this helper pipelines row chunks over three streams:
host->device copy of chunk i+1, quantise + GEMM of chunk i and device->host copy of chunk i-1
run concurrently, and the two copy directions overlap on the full-duplex link.  Several layers
that read the same activation (q/k/v fused, or any set sharing an input) are evaluated per
chunk so the activation crosses the link once.

Outputs are bit-identical to linear_vdm_w4a4 on the whole matrix: every output row depends only
on its own input row.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import torch

from . import _lib
from .kernels import vdm_w4a4 as vdm


class HostLinearLayer:
    """One W4A4 layer prepared for the pipeline (repacked weight, plain scales, fp16 bias)."""

    def __init__(self, qweight: torch.Tensor, wscales: torch.Tensor, bias_half: Optional[torch.Tensor] = None):
        self.n, k2 = qweight.shape
        self.k = 2 * k2
        self.w_b200, self.w_scale = vdm.prepare_b200_weight(qweight, wscales)
        self._keep = (qweight, wscales)
        self.bias = None if bias_half is None else bias_half.detach().half().contiguous()


class HostLinearPipeline:
    def __init__(self, device, k_max: int, n_max: int, chunk_rows: int = 4096, depth: int = 3,
                 act_dtype: torch.dtype = torch.float16):
        self.device = torch.device(device)
        self.chunk_rows, self.depth, self.act_dtype = chunk_rows, depth, act_dtype
        self.lib = _lib.load()
        self.ws_bytes = self.lib.b200w4a4_linear_workspace_bytes(chunk_rows, k_max)
        self.k_max, self.n_max = k_max, n_max
        dev = self.device
        self.xbuf = [torch.empty(chunk_rows * k_max, dtype=act_dtype, device=dev) for _ in range(depth)]
        self.obuf = [torch.empty(chunk_rows * n_max, dtype=torch.float16, device=dev) for _ in range(depth)]
        self.work = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(depth)]
        self.ev_x_free = [torch.cuda.Event() for _ in range(depth)]
        self.ev_cmp: List[torch.cuda.Event] = []
        self.ev_o_free: List[torch.cuda.Event] = []
        self._slot = 0            # output-buffer slot counter (one per layer per chunk)
        self._xslot = 0

    def _ensure_out_events(self):
        while len(self.ev_cmp) < self.depth:
            self.ev_cmp.append(torch.cuda.Event())
            self.ev_o_free.append(torch.cuda.Event())

    @torch.no_grad()
    def run(self, x_host: torch.Tensor, layers: Sequence[HostLinearLayer], outs_host: Sequence[torch.Tensor],
            clip_ratio: float = 1.0) -> None:
        """x_host [M,K] (pinned for real overlap), outs_host[i] [M,N_i] fp16 (pinned).  Returns after
        enqueueing; call synchronize() (or torch.cuda.synchronize()) before reading outs_host."""
        self.run_groups([(x_host, layers, outs_host)], clip_ratio)

    @torch.no_grad()
    def run_groups(self, groups: Sequence[tuple], clip_ratio: float = 1.0) -> None:
        """Several (x_host, layers, outs_host) groups, each as in run(), in one pipelined sequence: the
        copies and kernels of a group's first chunks overlap the tail of the group before it instead
        of waiting for it to drain (a step of a model is usually a few such groups, one per distinct
        activation matrix)."""
        for x_host, layers, outs_host in groups:
            m, k = x_host.shape
            assert x_host.dtype == self.act_dtype and k <= self.k_max and x_host.is_contiguous()
            for L, o in zip(layers, outs_host):
                assert L.k == k and o.shape == (m, L.n) and L.n <= self.n_max and o.dtype == torch.float16
        self._ensure_out_events()
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_stream(cur)
        dcode = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[self.act_dtype]
        for x_host, layers, outs_host in groups:
            m, k = x_host.shape
            for r0 in range(0, m, self.chunk_rows):
                rows = min(self.chunk_rows, m - r0)
                xb = self._xslot % self.depth
                self._xslot += 1
                xv = self.xbuf[xb][: rows * k].view(rows, k)
                with torch.cuda.stream(self.s_in):
                    self.s_in.wait_event(self.ev_x_free[xb])          # last compute on this x buffer is done
                    xv.copy_(x_host[r0:r0 + rows], non_blocking=True)
                    self.ev_in[xb].record(self.s_in)
                for L, o_host in zip(layers, outs_host):
                    ob = self._slot % self.depth
                    self._slot += 1
                    ov = self.obuf[ob][: rows * L.n].view(rows, L.n)
                    with torch.cuda.stream(self.s_cmp):
                        self.s_cmp.wait_event(self.ev_in[xb])
                        self.s_cmp.wait_event(self.ev_o_free[ob])     # previous D2H from this out buffer is done
                        rc = self.lib.b200w4a4_linear(
                            xv.data_ptr(), dcode, L.w_b200.data_ptr(), L.w_scale.data_ptr(),
                            L.bias.data_ptr() if L.bias is not None else None, ov.data_ptr(),
                            self.work.data_ptr(), self.ws_bytes, rows, L.n, k, float(clip_ratio),
                            ctypes.c_void_p(self.s_cmp.cuda_stream))
                        _lib.check(rc, "linear")
                        self.ev_cmp[ob].record(self.s_cmp)
                    with torch.cuda.stream(self.s_out):
                        self.s_out.wait_event(self.ev_cmp[ob])
                        o_host[r0:r0 + rows].copy_(ov, non_blocking=True)
                        self.ev_o_free[ob].record(self.s_out)
                with torch.cuda.stream(self.s_cmp):
                    self.ev_x_free[xb].record(self.s_cmp)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_cmp)

    def synchronize(self) -> None:
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.synchronize()
