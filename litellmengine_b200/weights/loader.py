"""Binding tensors to a model's parameters by name, and the random-weights mode.

A model declares what it wants as `{full tensor name: ParamSpec}`; a source offers
tensors by name.  `bind_weights` compares the two and raises ONE `WeightError`
that lists every missing tensor, every unexpected tensor and every wrong shape,
then hands each part its tensors.

Reference behaviour kept: binding by full name (src/model/qwen3.cpp:87-90,181-187,
859-877,1074-1088,1413-1416), shape checks against the configuration
(src/model/qwen3.cpp:92-105,189-218), an error for tensors nobody consumed
(src/main.cpp:161-165).  Different: a tied output head aliases the embedding
table when `lm_head.weight` is absent, where the reference throws
(src/model/qwen3.cpp:1417-1420).

Types: a tensor keeps the type it was stored in when that is bfloat16 or a 32-bit
float (a 32-bit tensor is never narrowed); float16 is widened to float32; integer
tensors become int32.  In the float32 run mode everything floating is widened to
float32, which is exact.
"""
from __future__ import annotations

import hashlib
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile, open_model_files, write_safetensors


class WeightError(ValueError):
    """Missing / unexpected tensors or wrong shapes, all listed in one message."""

    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights do not fit the model{(' (' + where + ')') if where else ''}:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {list(e)}, found {list(f)}" for n, e, f in self.wrong_shape))
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class ParamSpec:
    """What a part wants for one tensor.

    role 'matrix': an operand of a matrix product or a lookup table of vectors;
    kept in the stored type (bfloat16 or float32).  role 'scale': a small vector
    that multiplies in 32-bit (norm weights); always held as float32.  role
    'index': an integer table; held as int32.
    init: ('normal', std) or ('one_plus_normal', std) for the random-weights mode.
    optional_alias: name of another tensor to use when this one is absent.
    """
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple[str, float] = ("normal", 0.02)
    optional_alias: Optional[str] = None


class WeightSource:
    def names(self) -> List[str]:
        raise NotImplementedError

    def shape(self, name: str) -> Tuple[int, ...]:
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        raise NotImplementedError


class SafetensorsSource(WeightSource):
    """All tensors of a model folder's safetensors files."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._files = open_model_files(model_dir)
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self._files:
            for n in f.names():
                if n in self._where:
                    raise SafetensorsError(
                        f"tensor {n!r} is in both {self._where[n].path} and {f.path}")
                self._where[n] = f

    def names(self):
        return list(self._where)

    def shape(self, name):
        return self._where[name].shape(name)

    def get(self, name):
        return self._where[name].tensor(name)


class DictSource(WeightSource):
    def __init__(self, tensors: Dict[str, torch.Tensor]):
        self._t = dict(tensors)

    def names(self):
        return list(self._t)

    def shape(self, name):
        return tuple(self._t[name].shape)

    def get(self, name):
        return self._t[name]


def _name_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


_MASK32 = (1 << 32) - 1
_M1, _M2 = 0x7FEB352D, 0x846CA68B          # multipliers of a 32-bit integer finaliser ("lowbias32")


def _mix32(x: torch.Tensor) -> torch.Tensor:
    """A 32-bit avalanche hash on int64 tensors that hold values below 2^32: shifts, xors and
    products that stay below 2^63, so the host and the GPU compute the same integers."""
    x = x ^ (x >> 16)
    x = (x * _M1) & _MASK32
    x = x ^ (x >> 15)
    x = (x * _M2) & _MASK32
    return x ^ (x >> 16)


def seeded_normal(shape, key: int, std: float, mean: float, device, chunk: int = 1 << 24) -> torch.Tensor:
    """float32 tensor of `shape` whose element i is mean + std * z_i, z_i a function of (key, i) alone:
    the sum of eight 16-bit integers hashed from (key, i), centred and scaled to unit variance (an
    Irwin-Hall approximation of the normal distribution; |z| < 4.9).  Only integer arithmetic, one
    integer-to-float conversion and two float32 products are involved, so every device gives the same
    bits."""
    n = 1
    for d in shape:
        n *= int(d)
    out = torch.empty(n, dtype=torch.float32, device=device)
    k_lo, k_hi = key & _MASK32, (key >> 32) & _MASK32
    scale = (12.0 / (8.0 * (65536.0 ** 2 - 1.0))) ** 0.5
    for at in range(0, n, chunk):
        i = torch.arange(at, min(at + chunk, n), dtype=torch.int64, device=device)
        lo, hi = i & _MASK32, i >> 32
        total = torch.zeros_like(i)
        for word in range(4):                                    # four 32-bit hashes = eight 16-bit integers
            h = _mix32(_mix32(lo ^ k_lo ^ (word * 0x9E3779B9 & _MASK32)) ^ hi ^ k_hi)
            total += (h & 0xFFFF) + (h >> 16)
        z = (total - 262140).to(torch.float32) * scale            # 262140 = 8 * 65535 / 2
        out[at:at + z.numel()] = z * std + mean
    return out.view(tuple(shape))


class RandomSource(WeightSource):
    """Seeded random tensors for a set of `ParamSpec`s: matrices N(0, std), norm
    weights 1 + N(0, std).  Each tensor's values are a function of (seed, tensor name, element
    index), so they do not depend on which other tensors exist, and not on `device` either: drawn
    on the host or on the GPU, the same seed gives the same model, bit for bit (`seeded_normal`).
    Values are drawn in float32 and then rounded to `dtype`.
    Tensors that have an `optional_alias` (a tied output head) are left out.
    """

    def __init__(self, params: Dict[str, ParamSpec], seed: int, dtype: torch.dtype,
                 device: str = "cpu", include_aliased: bool = False):
        self._p = {n: p for n, p in params.items() if include_aliased or p.optional_alias is None}
        self.seed, self.dtype, self.device = seed, dtype, torch.device(device)

    def names(self):
        return list(self._p)

    def shape(self, name):
        return tuple(self._p[name].shape)

    def get(self, name):
        p = self._p[name]
        if p.role == "index":
            raise ValueError(f"{name}: no random rule for integer tables")
        kind, std = p.init
        if kind not in ("normal", "one_plus_normal"):
            raise ValueError(f"{name}: unknown init {kind!r}")
        t = seeded_normal(p.shape, _name_seed(self.seed, name), std, 1.0 if kind == "one_plus_normal" else 0.0, self.device)
        return t.to(self.dtype)


def _stored_to_held(name: str, t: torch.Tensor, role: str, run_dtype: torch.dtype) -> torch.Tensor:
    if role == "index":
        if t.dtype.is_floating_point:
            raise WeightError([], [], [], where=f"{name}: an integer table was stored as {t.dtype}")
        return t.to(torch.int32)
    if not t.dtype.is_floating_point:
        raise WeightError([], [], [], where=f"{name}: a floating tensor was stored as {t.dtype}")
    if role == "scale" or run_dtype == torch.float32:
        return t.to(torch.float32)
    if t.dtype == torch.bfloat16:
        return t
    return t.to(torch.float32)          # float32 stays; float16/float64 become float32


def check_source(params: Dict[str, ParamSpec], source: WeightSource, where: str = "") -> Dict[str, str]:
    """Compare what `source` offers with what the model wants.  Raises one `WeightError`
    naming all missing, unexpected and mis-shaped tensors.  Returns `{name: alias}` for the
    parameters that are absent but may use another tensor (a tied output head)."""
    have = set(source.names())
    missing, wrong, aliased = [], [], {}
    for name, p in params.items():
        if name not in have:
            if p.optional_alias is not None and p.optional_alias in params:
                aliased[name] = p.optional_alias
            else:
                missing.append(name)
            continue
        found = tuple(source.shape(name))
        if found != tuple(p.shape):
            wrong.append((name, tuple(p.shape), found))
    unexpected = sorted(have - set(params))
    if missing or unexpected or wrong:
        raise WeightError(sorted(missing), unexpected, wrong, where)
    return aliased


def fetch_tensor(source: WeightSource, name: str, p: ParamSpec, run_dtype: torch.dtype, device) -> torch.Tensor:
    """One tensor from the source, in the type it is held in, on `device`."""
    t = _stored_to_held(name, source.get(name), p.role, run_dtype)
    if t.device == torch.device(device):
        return t.clone() if t.device.type == "cpu" else t
    return t.to(device)


def bind_weights(params: Dict[str, ParamSpec], source: WeightSource, run_dtype: torch.dtype,
                 device, where: str = "") -> Dict[str, torch.Tensor]:
    """`check_source`, then every tensor on `device`.  An absent parameter with an alias maps
    to the SAME tensor object as its alias (no copy)."""
    aliased = check_source(params, source, where)
    out = {n: fetch_tensor(source, n, p, run_dtype, device) for n, p in params.items() if n not in aliased}
    for name, src in aliased.items():
        out[name] = out[src]
    return out


def write_random_model(config, model_dir: str, seed: int, dtype: torch.dtype = None,
                       device: str = "cpu") -> str:
    """The random-weights mode: write `config.json` and `model.safetensors` for
    `config` into `model_dir`, every tensor drawn from `RandomSource(seed)`.
    `dtype` defaults to the configuration's `torch_dtype`."""
    from ..config import save_config
    from ..parts.model import model_parameters
    if dtype is None:
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[getattr(config, "torch_dtype", "bfloat16")]
    params = model_parameters(config.plan())
    src = RandomSource(params, seed, dtype, device)
    tensors = {n: src.get(n) for n in src.names()}
    save_config(config, model_dir)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
