"""Weights by tensor name, checked as a whole against what the model expects.

vt-transformer loads one raw file a tensor and asserts on its byte size
(v1/models/qwen2-7b/inference_fp16.dag:87-142, v1/tensortype/cuda_tensor.cpp:102-111);
a missing file is a panic (v1/tensortype/common.hpp:72-75).  Here the names and shapes
of a folder are compared with the model's ``ParamSpec`` table before any data is read,
and every difference is reported in one ``WeightError``: missing tensors, tensors the
model does not know, wrong shapes and wrong kinds of dtype.

Tensors are handed out as they are stored: bfloat16 stays bfloat16, a tensor stored in
32-bit stays 32-bit; float16 and float64 (which no kernel reads) become bfloat16 and
float32; integer tables become int32.  What was converted is counted (``WeightSource.converted``) and
reported after loading (``load_report``): vt-transformer's own dump rounds everything to fp16 without a word
(v1/models/qwen2-7b/dump_from_huggingface.py:35).
"""
from __future__ import annotations

import fnmatch
import hashlib
from typing import Dict, Iterator, List, Mapping, Sequence, Tuple

import torch

from ..parts.base import ParamSpec
from . import safetensors_io as st

_FLOATS = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightError(ValueError):
    """The tensors of a model folder do not fit the model.  ``missing``, ``unexpected``,
    ``wrong_shape`` (name -> (expected, found)) and ``wrong_dtype`` (name -> (expected
    kind, found dtype)) say how."""

    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_dtype):
        self.where = where
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = dict(wrong_shape)
        self.wrong_dtype = dict(wrong_dtype)
        lines = [f"{where}: the tensors do not fit the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, (want, got) in sorted(self.wrong_shape.items()):
            lines.append(f"  wrong shape: {name} expected {list(want)}, found {list(got)}")
        for name, (want, got) in sorted(self.wrong_dtype.items()):
            lines.append(f"  wrong dtype: {name} expected {want}, found {got}")
        super().__init__("\n".join(lines))


class WeightSource:
    """Where tensors come from: ``entries()`` gives name -> (dtype, shape) without reading
    data, ``get(name)`` the tensor as stored."""

    where = "weights"
    converted: Dict[str, int]        # stored dtype -> tensors that ``get`` converted from it

    def entries(self) -> Dict[str, Tuple[torch.dtype, Tuple[int, ...]]]:
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def close(self) -> None:
        pass


class SafetensorsSource(WeightSource):
    def __init__(self, folder: str):
        self.where = folder
        self.index = st.index_folder(folder)
        self.files = st.MappedFiles()
        self.converted = {}

    def entries(self):
        return {n: (e.dtype, e.shape) for n, e in self.index.items()}

    def get(self, name: str) -> torch.Tensor:
        return normalise_dtype(self.files.tensor(self.index[name]), self.converted)

    def close(self) -> None:
        self.files.close()


class DictSource(WeightSource):
    def __init__(self, tensors: Mapping[str, torch.Tensor], where: str = "tensors"):
        self.tensors = tensors
        self.where = where
        self.converted = {}

    def entries(self):
        return {n: (t.dtype, tuple(t.shape)) for n, t in self.tensors.items()}

    def get(self, name: str) -> torch.Tensor:
        return normalise_dtype(self.tensors[name], self.converted)


def normalise_dtype(t: torch.Tensor, counts: Dict[str, int] = None) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if counts is not None:
        key = str(t.dtype).replace("torch.", "")
        counts[key] = counts.get(key, 0) + 1
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)          # round to nearest even; bfloat16's range holds float16's
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in _INTS:
        return t.to(torch.int32)
    raise TypeError(f"no kernel reads dtype {t.dtype}")


def load_report(source: "WeightSource", notes: Mapping[str, int], ignored: Sequence[str] = ()) -> Tuple[List[str], List[str]]:
    """(lines to tell, lines to warn of) about what loading changed: tensors converted by the source, matrices
    rounded from 32-bit or kept in it (``Runtime.notes``), tensors of the folder that the model does not read."""
    info, warn = [], []
    conv = getattr(source, "converted", None) or {}
    if conv.get("float16"):
        info.append(f"{source.where}: {conv['float16']} tensors stored in float16 were rounded to bfloat16 (to nearest even; "
                    f"no value can overflow or vanish, bfloat16's range holds float16's)")
    for key in sorted(k for k in conv if k != "float16"):
        info.append(f"{source.where}: {conv[key]} tensors stored in {key} were converted")
    if notes.get("rounded"):
        info.append(f"{source.where}: {notes['rounded']} matrices stored in float32 ({notes.get('rounded_values', 0):,} values) were "
                    f"rounded to bfloat16 (to nearest even): {notes.get('to_inf', 0)} values became infinite, "
                    f"{notes.get('to_zero', 0)} became zero")
    if notes.get("kept_fp32"):
        warn.append(f"{source.where}: {notes['kept_fp32']} matrices are stored in float32 and stay so: their products run the "
                    f"32-bit kernels, many times slower than the bfloat16 ones; fp32_weights='round' (--fp32-weights round) "
                    f"rounds them to bfloat16 at load")
    if ignored:
        warn.append(f"{source.where}: {len(ignored)} tensors that the model does not read were left aside: "
                    + ", ".join(sorted(ignored)[:6]) + (" ..." if len(ignored) > 6 else ""))
    return info, warn


def check_against(source: WeightSource, expected: Mapping[str, ParamSpec], ignored: Sequence[str] = ()) -> List[str]:
    """Raises one ``WeightError`` that lists every difference between the source and the
    model's parameter table.  Tensors whose names match a pattern of ``ignored`` (names that checkpoints of the
    architecture are known to carry and the model does not read) are no difference: they are returned."""
    found = source.entries()
    missing = [n for n, s in expected.items() if n not in found and not s.optional]
    aside = [n for n in found if n not in expected and any(fnmatch.fnmatchcase(n, pat) for pat in ignored)]
    unexpected = [n for n in found if n not in expected and n not in aside]
    wrong_shape, wrong_dtype = {}, {}
    for name, spec in expected.items():
        if name not in found:
            continue
        dtype, shape = found[name]
        if tuple(shape) != tuple(spec.shape):
            wrong_shape[name] = (tuple(spec.shape), tuple(shape))
        if spec.role == "table":
            if dtype not in _INTS:
                wrong_dtype[name] = ("an integer type", str(dtype))
        elif dtype not in _FLOATS:
            wrong_dtype[name] = ("a floating-point type", str(dtype))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(source.where, missing, unexpected, wrong_shape, wrong_dtype)
    return aside


# ----------------------------------------------------------------------------- random weights


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


# How the random-weights mode fills a tensor: ``ParamSpec.init`` names a function (shape, generator, sigma, device) ->
# float32 tensor.  A part whose tensors want another start registers one under a name of its own.
_INITIALISERS = {
    "normal": lambda shape, g, sigma, device: torch.randn(shape, generator=g, dtype=torch.float32, device=device) * sigma,
    "one_plus_normal": lambda shape, g, sigma, device: torch.randn(shape, generator=g, dtype=torch.float32,
                                                                   device=device) * sigma + 1.0,
    "zeros": lambda shape, g, sigma, device: torch.zeros(shape, dtype=torch.float32, device=device),
}


def register_initialiser(name: str, fn, replace: bool = False) -> None:
    """``fn(shape, generator, sigma, device)`` returns the float32 tensor that the random-weights mode stores (in
    bfloat16) for every ``ParamSpec`` whose ``init`` is ``name``."""
    if name in _INITIALISERS and not replace:
        raise ValueError(f"initialiser '{name}' is registered already")
    _INITIALISERS[name] = fn


def unregister_initialiser(name: str) -> None:
    _INITIALISERS.pop(name, None)


def random_tensor(name: str, spec: ParamSpec, seed: int, sigma: float, device="cpu") -> torch.Tensor:
    """The tensor ``name`` of a random model: N(0, sigma) for matrices and vectors,
    1 + N(0, sigma) for norm weights (or what the initialiser that ``spec.init`` names gives), stored in
    bfloat16; tables are zeros.  The numbers depend on (seed, name) only, not on the order in which tensors
    are made."""
    if spec.role == "table":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    try:
        fill = _INITIALISERS[spec.init]
    except KeyError:
        raise ValueError(f"unknown initialiser '{spec.init}' for {name}; known: {', '.join(sorted(_INITIALISERS))}") from None
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, name))
    return fill(tuple(spec.shape), g, sigma, device).to(torch.bfloat16)


class RandomSource(WeightSource):
    """Seeded random weights made on demand (on ``device``), never all at once."""

    def __init__(self, expected: Mapping[str, ParamSpec], seed: int, sigma: float, device="cpu"):
        self.expected = {n: s for n, s in expected.items() if not s.optional}
        self.seed, self.sigma, self.device = seed, sigma, device
        self.converted = {}
        self.where = f"random weights (seed {seed}, sigma {sigma})"

    def entries(self):
        return {n: (torch.int32 if s.role == "table" else torch.bfloat16, tuple(s.shape))
                for n, s in self.expected.items()}

    def get(self, name: str) -> torch.Tensor:
        return random_tensor(name, self.expected[name], self.seed, self.sigma, self.device)


def iter_source(source: WeightSource) -> Iterator[Tuple[str, torch.Tensor]]:
    for name in source.entries():
        yield name, source.get(name)
