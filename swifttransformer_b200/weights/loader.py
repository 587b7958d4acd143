"""Fill a model's parameters from a folder of safetensors, by tensor name.

One pass compares what the model asks for (its ``ParamSpec`` list) with what
the files hold and raises ONE error that lists every missing tensor, every
unexpected tensor and every wrong shape.  Storage types: matrices and lookup
tables in the compute dtype (bfloat16 or float32), vectors (biases, norm
weights) always in 32-bit, integer tables in int32; a bfloat16 value widened
to 32-bit is exact, so both compute dtypes see the same numbers.

Reference behaviour for comparison: one file per tensor, first problem aborts
(src/csrc/model/gpt/gpt_weight.cc:193-250, 258-326).
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional

import torch

from .safetensors_io import SafetensorsError, open_model_files
from .spec import ParamSpec


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every mismatch."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong
        lines = [f"weights in '{where}' do not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or type ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def load_named_tensors(
    model_dir: str,
    specs: Iterable[ParamSpec],
    compute_dtype: torch.dtype,
    device: torch.device,
    canonical_name: Optional[Callable[[str], Optional[str]]] = None,
) -> Dict[str, torch.Tensor]:
    """Return ``spec.name -> device tensor`` for every spec.

    ``canonical_name`` maps a name found in the files to the name the specs use
    (or to None for a tensor that is to be ignored, such as a version marker).
    """
    specs = list(specs)
    files = open_model_files(model_dir)
    found = {}
    for f in files:
        for raw in f.names():
            name = canonical_name(raw) if canonical_name else raw
            if name is None:
                continue
            if name in found:
                raise SafetensorsError(f"tensor '{name}' occurs twice in '{model_dir}'")
            found[name] = (f, raw)

    by_name = {s.name: s for s in specs}
    missing, wrong = [], []
    for s in specs:
        if s.name not in found:
            if s.tied_to is None:
                missing.append(s.name)
            continue
        f, raw = found[s.name]
        info = f.tensors[raw]
        if tuple(info.shape) != tuple(s.shape):
            wrong.append(f"{s.name}: file has {list(info.shape)}, model wants {list(s.shape)}")
        elif info.dtype.is_floating_point == (s.role == "int_table"):
            wrong.append(f"{s.name}: file has {info.dtype}, model wants "
                         f"{'an integer' if s.role == 'int_table' else 'a floating-point'} tensor")
    unexpected = sorted(n for n in found if n not in by_name)
    if missing or unexpected or wrong:
        raise WeightError(model_dir, missing, unexpected, wrong)

    out: Dict[str, torch.Tensor] = {}
    for s in specs:
        if s.name not in found:
            continue
        f, raw = found[s.name]
        t = f.get(raw)
        out[s.name] = t.to(device=device, dtype=s.storage_dtype(compute_dtype, t.dtype)).contiguous()
    for s in specs:
        if s.name not in out:
            out[s.name] = out[s.tied_to]          # alias, not a copy
        elif s.tied_to is not None and s.tied_to in out:
            # a tied tensor that the file repeats must repeat it exactly
            if not torch.equal(out[s.name], out[s.tied_to]):
                raise WeightError(model_dir, [], [], [
                    f"{s.name}: differs from '{s.tied_to}' although the configuration ties them"])
            out[s.name] = out[s.tied_to]
    for f in files:
        f.close()
    return out
