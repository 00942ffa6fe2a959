"""Model export: TorchScript always, ONNX when the ``onnx`` package is importable (reference: ``core/classes/exportable.py:39``,
``utils/export_utils.py``).  A model (or module) mixes in ``Exportable`` and provides ``input_example()``; ``export()`` puts the
module in eval mode, freezes it, traces it and verifies the traced outputs against eager outputs."""
from __future__ import annotations

import os
from typing import Any, List, Optional, Sequence, Tuple

import torch


def verify_runtime(module: torch.nn.Module, traced, example: Tuple, rtol: float = 1e-3, atol: float = 1e-4) -> bool:
    with torch.no_grad():
        a = module(*example)
        b = traced(*example)
    a = a if isinstance(a, (tuple, list)) else (a,)
    b = b if isinstance(b, (tuple, list)) else (b,)
    return all(torch.allclose(x.float(), y.float(), rtol=rtol, atol=atol) for x, y in zip(a, b) if torch.is_tensor(x))


class Exportable:
    @property
    def input_module(self):
        return self

    @property
    def output_module(self):
        return self

    def input_example(self, max_batch: int = 1, max_dim: int = 256):
        raise NotImplementedError("provide input_example() to make the module exportable")

    def _prepare_for_export(self, **kw) -> None:
        self.eval()
        for p in self.parameters():
            p.requires_grad_(False)

    def export(self, output: str, input_example: Optional[Sequence[Any]] = None, verbose: bool = False, check_trace: bool = True,
               dynamic_axes: Optional[dict] = None, onnx_opset_version: Optional[int] = None, **kw) -> Tuple[List[str], List[str]]:
        self._prepare_for_export(**kw)
        example = tuple(input_example) if input_example is not None else tuple(self.input_example())
        ext = os.path.splitext(output)[1].lower()
        fwd = getattr(self, "forward_for_export", None)
        module = self
        if fwd is not None:
            class _Wrap(torch.nn.Module):
                def __init__(self, m):
                    super().__init__()
                    self.m = m

                def forward(self, *a):
                    return self.m.forward_for_export(*a)

            module = _Wrap(self)
        if ext in (".pt", ".ts"):
            traced = torch.jit.trace(module, example, check_trace=False, strict=False)
            if check_trace and not verify_runtime(module, traced, example):
                raise RuntimeError("the traced module disagrees with the eager module on the example input")
            traced.save(output)
            return [output], [f"TorchScript module traced with {len(example)} inputs"]
        if ext == ".onnx":
            try:
                import onnx  # noqa: F401
            except ImportError as e:
                raise RuntimeError("ONNX export needs the 'onnx' package, which is not installed") from e
            torch.onnx.export(module, example, output, opset_version=onnx_opset_version or 17, dynamic_axes=dynamic_axes, verbose=verbose)
            return [output], ["ONNX graph"]
        raise ValueError(f"unsupported export format '{ext}' (use .pt / .ts / .onnx)")
