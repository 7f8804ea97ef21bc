"""Host-side objects of the MoE expert path: an expert bank resident in HBM, one
MoE-FFN layer (the reference's Model::moe, src/model/model.cpp:399-510, with the
ffn RMSNorm before it and the residual add after it) and the resident
whole-stack decode loop (tools/bench/q4k_stream_ffn.hip:1233-1325 run_resident).
All arithmetic is done by libknj_device.so."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import synth
from ._lib import DT_BF16, DT_F32, MoeFfnArgs, check, lib

_DT = {torch.float32: DT_F32, torch.bfloat16: DT_BF16}


@dataclass
class ExpertBank:
    """Weights of one MoE layer, all on one device.

    gate, up: uint8 [E][F][H/256][144]; down: uint8 [E][H][F/256][144] (Q4_K) or [...][210] (Q6_K);
    router: bf16 [E][H]; router_bias: f32 [E] or None; norm_w: bf16 [H] or None.
    """
    gate: torch.Tensor
    up: torch.Tensor
    down: torch.Tensor
    router: torch.Tensor
    router_bias: torch.Tensor | None = None
    norm_w: torch.Tensor | None = None
    rms_eps: float = synth.RMS_EPS

    @property
    def n_experts(self) -> int:
        return self.gate.shape[0]

    @property
    def ffn(self) -> int:
        return self.gate.shape[1]

    @property
    def hidden(self) -> int:
        return self.gate.shape[2] * 256

    def nbytes(self) -> int:
        return self.gate.numel() + self.up.numel() + self.down.numel()

    @staticmethod
    def from_numpy(bank: dict, router_bits: np.ndarray, bias: np.ndarray | None = None,
                   norm_bits: np.ndarray | None = None, device="cuda") -> "ExpertBank":
        def bf(bits):
            return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(device)
        return ExpertBank(
            gate=torch.from_numpy(bank["gate"]).to(device), up=torch.from_numpy(bank["up"]).to(device),
            down=torch.from_numpy(bank["down"]).to(device), router=bf(router_bits),
            router_bias=None if bias is None else torch.from_numpy(bias).to(device),
            norm_w=None if norm_bits is None else bf(norm_bits))

    @staticmethod
    def random(n_experts: int = synth.N_EXPERTS, hidden: int = synth.HIDDEN, ffn: int = synth.FFN, seed: int = 0,
               with_norm: bool = True, device="cuda") -> "ExpertBank":
        """Random-init bank drawn on the device (for large resident stacks): same
        value distributions as synth.q4k_rows, torch's CUDA generator."""
        g = torch.Generator(device=device)
        g.manual_seed(seed)

        def q4k(rows, n_in):
            nb = n_in // 256
            blk = torch.randint(0, 256, (n_experts, rows, nb, 144), dtype=torch.uint8, device=device, generator=g)
            dd = (torch.randn((n_experts, rows, nb, 2), device=device, generator=g).abs() * 0.01).to(torch.float16)
            blk[..., 0:4] = dd.view(torch.uint8).reshape(n_experts, rows, nb, 4)
            return blk
        router = (torch.randn((n_experts, hidden), device=device, generator=g) * 0.02).to(torch.bfloat16)
        norm = (1.0 + 0.02 * torch.randn(hidden, device=device, generator=g)).to(torch.bfloat16) if with_norm else None
        return ExpertBank(gate=q4k(ffn, hidden), up=q4k(ffn, hidden), down=q4k(hidden, ffn), router=router, norm_w=norm)


class MoeFfnLayer:
    """One MoE-FFN layer bound to a maximum token count (workspace is allocated
    once here; calls allocate nothing)."""

    def __init__(self, bank: ExpertBank, top_k: int = synth.TOP_K, max_tokens: int = 64, residual: bool = False,
                 use_norm: bool = True, workspace: torch.Tensor | None = None):
        self.bank, self.top_k, self.max_tokens, self.residual = bank, top_k, max_tokens, residual
        self.use_norm = use_norm and bank.norm_w is not None
        need = max(lib().knj_moe_ffn_workspace_bytes(max_tokens, bank.hidden, bank.ffn, bank.n_experts, top_k, mode)
                   for mode in (0, 1))
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.uint8, device=bank.gate.device)
        assert workspace.numel() >= need and workspace.data_ptr() % 256 == 0
        self.workspace = workspace
        self._need = need

    def _args(self, x: torch.Tensor, out: torch.Tensor, taps=None, fused_combine: bool = False) -> MoeFfnArgs:
        b = self.bank
        T, H = x.shape
        assert H == b.hidden and T <= self.max_tokens and x.is_contiguous() and out.is_contiguous()
        a = MoeFfnArgs()
        a.n_tokens, a.hidden, a.ffn, a.n_experts, a.top_k = T, H, b.ffn, b.n_experts, self.top_k
        a.x_dtype, a.x, a.ldx = _DT[x.dtype], x.data_ptr(), H
        a.w_router = b.router.data_ptr()
        a.router_bias = b.router_bias.data_ptr() if b.router_bias is not None else None
        a.w_gate, a.w_up, a.w_down = b.gate.data_ptr(), b.up.data_ptr(), b.down.data_ptr()
        a.down_format = 1 if b.down.shape[-1] == 210 else 0  # Q6_K down matrices of a mixed-format layer
        a.norm_w = b.norm_w.data_ptr() if self.use_norm else None
        a.rms_eps = b.rms_eps
        a.residual = 1 if self.residual else 0
        a.fused_combine = 1 if fused_combine else 0
        a.out, a.out_dtype, a.ldo = out.data_ptr(), _DT[out.dtype], H
        a.workspace, a.workspace_bytes = self.workspace.data_ptr(), self.workspace.numel()
        if taps is not None:
            a.tap_pair_exp, a.tap_pair_w = taps[0].data_ptr(), taps[1].data_ptr()
        return a

    def _run(self, fn, x, out, out_dtype, return_routing, fused_combine=False):
        if out is None:
            out = torch.empty(x.shape, dtype=out_dtype or torch.float32, device=x.device)
        taps = None
        if return_routing:
            P = x.shape[0] * self.top_k
            taps = (torch.empty(P, dtype=torch.int32, device=x.device), torch.empty(P, dtype=torch.float32, device=x.device))
        args = self._args(x, out, taps, fused_combine)
        check(fn(C.byref(args), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return (out, taps[0], taps[1]) if return_routing else out

    def decode(self, x, out=None, out_dtype=None, return_routing=False):
        """f32-accurate path (batch <= 64 is the intended use)."""
        return self._run(lib().knj_moe_ffn_decode_launch, x, out, out_dtype, return_routing)

    def prefill(self, x, out=None, out_dtype=None, return_routing=False, fused_combine=False):
        """Grouped-GEMM path over per-expert token buckets. fused_combine=False: per-pair rows + the ordered combine
        kernel (reproducible, and the faster form); True: the weighted sum fused into the down GEMM's epilogue
        (f32 reductions, unordered)."""
        return self._run(lib().knj_moe_ffn_prefill_launch, x, out, out_dtype, return_routing, fused_combine)


class MoeStack:
    """The resident whole-stack loop: L layers, each RMSNorm -> MoE -> residual
    add, the residual stream kept in bf16 between layers."""

    def __init__(self, banks: list[ExpertBank], top_k: int = synth.TOP_K, max_tokens: int = 64):
        need = max(lib().knj_moe_ffn_workspace_bytes(max_tokens, b.hidden, b.ffn, b.n_experts, top_k, 0) for b in banks)
        self.workspace = torch.empty(need, dtype=torch.uint8, device=banks[0].gate.device)
        self.layers = [MoeFfnLayer(b, top_k, max_tokens, residual=True, use_norm=True, workspace=self.workspace)
                       for b in banks]
        self.max_tokens = max_tokens
        self._buf = None
        self._graph = None

    def step(self, x: torch.Tensor) -> torch.Tensor:
        """x bf16 [B][H] -> residual stream after the last layer (bf16). Eager launches."""
        B, H = x.shape
        if self._buf is None or self._buf[0].shape != x.shape:
            self._buf = (torch.empty_like(x), torch.empty_like(x))
            self._graph = None
        cur = x
        for i, layer in enumerate(self.layers):
            nxt = self._buf[i & 1]
            layer.decode(cur, out=nxt)
            cur = nxt
        return cur

    def capture(self, x: torch.Tensor):
        """Capture one whole-stack step over the static input buffer `x` into a
        CUDA graph; returns (graph, output tensor). Replays read x in place."""
        self.step(x)  # warm-up: set function attributes, allocate ping-pong buffers
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self.step(x)
        return g, out


class FusedMoeStack:
    """The resident stack for a decode batch of 1..64 tokens as ONE cooperative launch (knj_moe_stack_*): the per-layer loop,
    its routing and its hand-offs run inside a single kernel with grid barriers between the stages. Buffers are
    static: write the step's rows into `self.x` (or pass them to step) and read `self.out` after the launch."""

    def __init__(self, banks: list[ExpertBank], top_k: int = synth.TOP_K, n_tokens: int = 1, dtype=torch.bfloat16,
                 residual: bool = True, use_norm: bool = True, taps: bool = False,
                 layer_inputs: list[torch.Tensor] | None = None, keep_outputs: bool = False):
        """layer_inputs: one [n_tokens][H] tensor per layer that the layer reads INSTEAD of its predecessor's output
        (independent layers, e.g. to drive every layer with fresh rows); default: the layers form a chain.
        keep_outputs: every layer writes a buffer of its own (self.outs[l]) instead of two alternating ones."""
        dev = banks[0].gate.device
        H = banks[0].hidden
        self.x = torch.zeros((n_tokens, H), dtype=dtype, device=dev)
        self._buf = (torch.zeros_like(self.x), torch.zeros_like(self.x))
        self.outs = [torch.zeros_like(self.x) for _ in banks] if keep_outputs else None
        ws = torch.empty(256, dtype=torch.uint8, device=dev)
        self._layers = [MoeFfnLayer.__new__(MoeFfnLayer) for _ in banks]
        P = n_tokens * top_k
        self.taps = [(torch.empty(P, dtype=torch.int32, device=dev), torch.empty(P, dtype=torch.float32, device=dev))
                     for _ in banks] if taps else None
        arr = (MoeFfnArgs * len(banks))()
        cur = self.x
        for l, (layer, b) in enumerate(zip(self._layers, banks)):
            layer.bank, layer.top_k, layer.max_tokens, layer.residual = b, top_k, n_tokens, residual
            layer.use_norm = use_norm and b.norm_w is not None
            layer.workspace = ws
            nxt = self.outs[l] if keep_outputs else self._buf[l & 1]
            if layer_inputs is not None:
                cur = layer_inputs[l]
            arr[l] = layer._args(cur, nxt, self.taps[l] if taps else None)
            cur = nxt
        self.out = cur
        self._banks, self._inputs = banks, layer_inputs  # keep the weights and the rows alive
        h = C.c_void_p()
        check(lib().knj_moe_stack_create(arr, len(banks), C.byref(h)))
        self._h = h

    def step(self, x: torch.Tensor | None = None) -> torch.Tensor:
        if x is not None:
            self.x.copy_(x)
        check(lib().knj_moe_stack_decode_launch(self._h, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return self.out

    def status(self) -> None:
        """Waits for the stream; raises if a grid barrier of the last launches gave up."""
        check(lib().knj_moe_stack_status(self._h, C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def set_wait(self, wait_cycles: int = 0, stall_first_barrier: int = 0) -> None:
        """Limit of the kernel's bounded waits (SM cycles; 0 = default) and the test hook that makes the first
        grid barrier unreachable."""
        check(lib().knj_moe_stack_set_wait(self._h, wait_cycles, stall_first_barrier))

    def close(self):
        if self._h:
            lib().knj_moe_stack_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
