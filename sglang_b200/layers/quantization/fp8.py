"""``Fp8Config`` / ``Fp8LinearMethod`` for block-quantised checkpoints
(``python/sglang/srt/layers/quantization/fp8.py:95-178,205-499``), restricted to what the
block-FP8 W8A8 path needs: e4m3 weights ``[N, K]`` with fp32 ``weight_scale_inv
[ceil(N/128), ceil(K/128)]`` and dynamic per-token-group activation quantisation."""

from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch
from torch.nn import Module, Parameter

from .fp8_utils import dispatch_w8a8_block_fp8_linear


class Fp8Config:
    """Quantisation config of a block-FP8 checkpoint (``fp8.py:95-178``)."""

    def __init__(self, is_checkpoint_fp8_serialized: bool = True, activation_scheme: str = "dynamic",
                 weight_block_size: Optional[List[int]] = None, requant_weight_ue8m0: bool = False):
        if activation_scheme != "dynamic":
            raise ValueError("The block-wise quantization only supports dynamic activation scheme for now.")
        if weight_block_size is None:
            weight_block_size = [128, 128]
        if not is_checkpoint_fp8_serialized:
            raise ValueError("The block-wise quantization only supports fp8-serialized checkpoint for now.")
        if len(weight_block_size) != 2 or list(weight_block_size) != [128, 128]:
            raise ValueError(f"weight_block_size must be [128, 128], got {weight_block_size}.")
        self.is_checkpoint_fp8_serialized = True
        self.activation_scheme = activation_scheme
        self.weight_block_size = list(weight_block_size)
        # Requantise weights whose block scales are not powers of two to UE8M0 scales at load time, as the reference
        # does for its Blackwell DeepGEMM path (fp8_utils.py:416-507); changes the weight codes, so results move by
        # the requantisation error.  Off by default: such weights then use the fp32-scale GEMM, which is exact.
        self.requant_weight_ue8m0 = requant_weight_ue8m0

    @classmethod
    def get_name(cls) -> str:
        return "fp8"

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "Fp8Config":
        """Read ``quantization_config`` of a HF checkpoint (``fp8.py:167-178``)."""
        quant_method = config.get("quant_method", "fp8")
        return cls(is_checkpoint_fp8_serialized="fp8" in quant_method,
                   activation_scheme=config.get("activation_scheme", "dynamic"),
                   weight_block_size=config.get("weight_block_size"))


class Fp8LinearMethod:
    """Linear method for block-FP8 W8A8 (``fp8.py:205-499``): ``create_weights`` registers the
    parameters the loader fills, ``apply`` runs quant + GEMM on the current stream."""

    def __init__(self, quant_config: Fp8Config, tp_size: int = 1):
        self.quant_config = quant_config
        self.block_quant = True
        self.tp_size = tp_size
        self.w8a8_block_fp8_linear = dispatch_w8a8_block_fp8_linear()

    def create_weights(self, layer: Module, input_size_per_partition: int, output_partition_sizes: List[int],
                       input_size: int, output_size: int, params_dtype: torch.dtype, **extra_weight_attrs):
        output_size_per_partition = sum(output_partition_sizes)
        block_n, block_k = self.quant_config.weight_block_size
        tp_size = self.tp_size
        # required by row parallel (fp8.py:251-258)
        if tp_size > 1 and input_size // input_size_per_partition == tp_size:
            if input_size_per_partition % block_k != 0:
                raise ValueError(f"Weight input_size_per_partition = {input_size_per_partition} is not divisible by "
                                 f"weight quantization block_k = {block_k}.")
        # required by column parallel or merged weights (fp8.py:259-269)
        if (tp_size > 1 and output_size // output_size_per_partition == tp_size) or len(output_partition_sizes) > 1:
            for size in output_partition_sizes:
                if size % block_n != 0:
                    raise ValueError(f"Weight output_partition_size = {size} is not divisible by "
                                     f"weight quantization block_n = {block_n}.")
        layer.logical_widths = output_partition_sizes
        layer.input_size_per_partition = input_size_per_partition
        layer.output_size_per_partition = output_size_per_partition
        layer.orig_dtype = params_dtype
        device = extra_weight_attrs.get("device")
        weight = Parameter(torch.empty(output_size_per_partition, input_size_per_partition, dtype=torch.float8_e4m3fn,
                                       device=device), requires_grad=False)
        layer.register_parameter("weight", weight)
        scale = Parameter(torch.full(((output_size_per_partition + block_n - 1) // block_n,
                                      (input_size_per_partition + block_k - 1) // block_k),
                                     torch.finfo(torch.float32).min, dtype=torch.float32, device=device),
                          requires_grad=False)
        layer.register_parameter("weight_scale_inv", scale)
        layer.register_parameter("input_scale", None)

    def process_weights_after_loading(self, layer: Module) -> None:
        """Pick the GEMM for this layer once the weights are in place (``fp8.py:340-363``; the UE8M0 handling
        mirrors ``fp8_utils.py:416-507``).  If every block scale is a power of two (a UE8M0 checkpoint), or after
        ``requant_weight_ue8m0``, the exponents are packed for the tensor core's block-scaling path; otherwise the
        layer keeps the fp32-scale GEMM.  One host synchronisation, at load time only."""
        from .fp8_kernel import pack_ue8m0_scales
        from .fp8_utils import requant_weight_ue8m0
        layer.weight_scale_ue8m0 = None
        ws = layer.weight_scale_inv.data
        if not ws.is_cuda:
            return None
        bits = ws.contiguous().view(torch.int32)
        pow2 = bool(((bits & 0x7FFFFF) == 0).all()) and bool((bits > 0).all())
        if not pow2 and self.quant_config.requant_weight_ue8m0:
            wq, ws = requant_weight_ue8m0(layer.weight.data, ws, self.quant_config.weight_block_size)
            layer.weight.data = wq
            layer.weight_scale_inv.data = ws
            pow2 = True
        if pow2:
            layer.weight_scale_ue8m0 = pack_ue8m0_scales(ws)
        return None

    def apply(self, layer: Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``Fp8LinearMethod.apply`` (``fp8.py:453-499``, block-quant branch ``:482-489``)."""
        packed = getattr(layer, "weight_scale_ue8m0", None)
        if packed is not None:
            from .fp8_utils import w8a8_block_fp8_linear_ue8m0
            return w8a8_block_fp8_linear_ue8m0(x, layer.weight, packed, bias)
        return self.w8a8_block_fp8_linear(input=x, weight=layer.weight,
                                          block_size=self.quant_config.weight_block_size,
                                          weight_scale=layer.weight_scale_inv, input_scale=None, bias=bias)
