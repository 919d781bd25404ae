"""Grouped expert MLPs: rows of local expert e (contiguous, `tokens_per_expert[e]` of them)
go through fc1 -> activation -> (x routed probability) -> fc2 with that expert's weights.

Parity: `TorchGroupedExperts` / `TransformerEngineGroupedExperts` / `build_experts` of
`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:467-628`: weights
`weight1[E_local, fc1_out, H]`, `weight2[E_local, H, F]`, N(0, 0.02) init, no bias;
`fc1_out = 2F` for swiglu (gate first, linear second); probability applied after the
activation and before fc2.

Backends
  "torch"   : per-expert `F.linear` loop (the PyTorch oracle; differentiable).
  "tcgen05" : this library's grouped GEMM kernels (csrc/gemm), tile scheduling driven by
              device-side counts, SwiGLU x prob fused into fc1's epilogue.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.nn.functional as F

ACTIVATIONS = ("swiglu", "gelu", "silu", "relu")


def activate(x: torch.Tensor, activation: str) -> torch.Tensor:
    if activation == "swiglu":
        gate, lin = torch.chunk(x, 2, dim=-1)
        return F.silu(gate) * lin
    if activation == "gelu":
        return F.gelu(x)
    if activation == "silu":
        return F.silu(x)
    if activation == "relu":
        return F.relu(x)
    raise ValueError(f"unsupported activation {activation!r}; expected one of {ACTIVATIONS}")


class GroupedExpertsBase(torch.nn.Module):
    def __init__(self, num_local_experts: int, hidden_size: int, ffn_hidden_size: int,
                 dtype: torch.dtype = torch.bfloat16, activation: str = "swiglu", device="cuda",
                 init_std: float = 0.02):
        super().__init__()
        if activation not in ACTIVATIONS:
            raise ValueError(f"unsupported activation {activation!r}")
        self.activation = activation
        self.gated = activation == "swiglu"
        self.num_local_experts, self.hidden_size, self.ffn_hidden_size = num_local_experts, hidden_size, ffn_hidden_size
        fc1_out = 2 * ffn_hidden_size if self.gated else ffn_hidden_size
        self.weight1 = torch.nn.Parameter(torch.empty(num_local_experts, fc1_out, hidden_size, dtype=dtype, device=device))
        self.weight2 = torch.nn.Parameter(torch.empty(num_local_experts, hidden_size, ffn_hidden_size, dtype=dtype, device=device))
        torch.nn.init.normal_(self.weight1, mean=0.0, std=init_std)
        torch.nn.init.normal_(self.weight2, mean=0.0, std=init_std)


class TorchGroupedExperts(GroupedExpertsBase):
    """Reference math with library GEMMs; one host read of the split sizes per call."""

    def forward(self, hidden_states: torch.Tensor, tokens_per_expert, routed_probs: torch.Tensor) -> torch.Tensor:
        splits = [int(v) for v in (tokens_per_expert.tolist() if torch.is_tensor(tokens_per_expert) else tokens_per_expert)]
        H = self.weight2.shape[1]
        if sum(splits) == 0:
            return hidden_states.new_empty((0, H))
        outs = []
        xs = torch.split(hidden_states[:sum(splits)], splits)
        ps = torch.split(routed_probs[:sum(splits)].to(torch.float32), splits)
        for e, (x, p) in enumerate(zip(xs, ps)):
            if x.shape[0] == 0:
                continue
            inter = activate(F.linear(x, self.weight1[e]), self.activation)
            inter = (inter * p[:, None]).to(x.dtype)
            outs.append(F.linear(inter, self.weight2[e]))
        return torch.cat(outs, 0)


def build_experts(backend: str, num_local_experts: int, hidden_size: int, ffn_hidden_size: int,
                  dtype: torch.dtype, activation: str, device="cuda", use_fp8: bool = False) -> Tuple[torch.nn.Module, str]:
    """backend: 'auto' | 'tcgen05' | 'torch' ('te' is accepted as an alias of 'auto': the library
    grouped GEMM of the reference is replaced by this repository's own kernels)."""
    if backend in ("auto", "tcgen05", "te"):
        try:
            from .experts_tcgen05 import Tcgen05GroupedExperts
            return (Tcgen05GroupedExperts(num_local_experts, hidden_size, ffn_hidden_size, dtype, activation, device,
                                          use_fp8=use_fp8),
                    "tcgen05_grouped_gemm")
        except Exception as exc:  # unsupported shape/dtype or extension not built
            if backend == "tcgen05":
                raise
            import warnings
            warnings.warn(f"tcgen05 grouped experts unavailable ({exc}); using the torch fallback")
    elif backend != "torch":
        raise ValueError("expert backend must be auto, tcgen05, te or torch")
    return TorchGroupedExperts(num_local_experts, hidden_size, ffn_hidden_size, dtype, activation, device), "torch_fallback"
