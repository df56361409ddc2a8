"""Weights by tensor name: what the model expects against what the files hold.

The model says which tensors it wants (`expected`: name -> shape).  `check` compares that with
the tensors found and raises ONE error that lists everything wrong at once: missing names,
unexpected names, and wrong shapes.  `keep_dtype` is the storage policy: bfloat16 stays bfloat16,
a tensor stored in 32 bits stays in 32 bits, float16 stays as stored (it has more mantissa bits
than bfloat16: a float32 engine widens it exactly, as adarsh-sgh/edgelm's exporter does,
tools/export.py:35, and a bfloat16 engine rounds it once), 64-bit floats become float32, and
integer tables become int32.  What precision a part computes in is the part's decision, taken
when it receives its tensors.
"""
import torch

from . import safetensors_io
from .errors import WeightsError


def keep_dtype(t):
    if t.dtype in (torch.bfloat16, torch.float16, torch.float32, torch.int32):
        return t
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8, torch.bool):
        return t.to(torch.int32)
    raise WeightsError(f"dtype {t.dtype} is not kept")


def check(expected, found, ignorable=()):
    """Raise one WeightsError naming every missing, unexpected and misshapen tensor."""
    missing = [n for n in expected if n not in found]
    unexpected = [n for n in found if n not in expected and n not in ignorable]
    wrong = [(n, tuple(found[n].shape), tuple(expected[n])) for n in expected
             if n in found and tuple(found[n].shape) != tuple(expected[n])]
    if not (missing or unexpected or wrong):
        return
    lines = ["the weights do not fit the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " + ", ".join(f"{n} is {list(f)}, expected {list(e)}" for n, f, e in sorted(wrong)))
    err = WeightsError("\n".join(lines))
    err.missing, err.unexpected, err.wrong_shape = sorted(missing), sorted(unexpected), sorted(wrong)
    raise err


def load_checked(model_dir, expected, ignorable=()):
    """name -> CPU tensor for every expected name, after the check, in the kept dtype."""
    found = safetensors_io.read_dir(model_dir)
    check(expected, found, ignorable)
    return {n: keep_dtype(found[n]) for n in expected}
