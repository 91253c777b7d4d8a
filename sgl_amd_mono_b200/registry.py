"""The monokernel spec interface that SGLang holds, with a stand-in for when SGLang is absent.

The reference only consumes this interface (``sgl_amd_mono/__init__.py:44-54`` imports
``register`` from ``sglang.kernels.plugin_kernels.amd.spec`` or
``sglang.srt.monokernels.spec``; ``glm53/spec.py:33-52`` imports ``DeviceLimits, Feature,
MonoSpec, Numerics, NumericsKind, Requirements``; ``test/unit/test_glm53_spec.py:46-68``
uses ``registry.ShapeKey``, ``find_spec`` and ``spec_registered``).  When SGLang is
importable its own types are re-exported; otherwise the classes below carry the same
names, fields and behaviour as far as the reference's uses show them, so that specs,
tests and the stand-alone runner work without a server.
"""

from __future__ import annotations

import enum
import importlib
from dataclasses import dataclass, field
from typing import Any, Callable

def _sglang_spec_module():
    """SGLang's monokernel spec module: the reference tries these two locations in this order
    (``sgl_amd_mono/__init__.py:46-49``).  None when SGLang is not installed."""
    for name in ("sglang.kernels.plugin_kernels.amd.spec", "sglang.srt.monokernels.spec"):
        try:
            return importlib.import_module(name)
        except ModuleNotFoundError:
            continue
    return None


_sgl = _sglang_spec_module()
HAVE_SGLANG = _sgl is not None
if HAVE_SGLANG:  # pragma: no cover - SGLang is not installed in the build environment
    DeviceLimits, Feature, MonoSpec, Numerics = _sgl.DeviceLimits, _sgl.Feature, _sgl.MonoSpec, _sgl.Numerics
    NumericsKind, Requirements, register = _sgl.NumericsKind, _sgl.Requirements, _sgl.register
    _sgl_registry = importlib.import_module(_sgl.__name__.rsplit(".", 1)[0] + ".registry")
    ShapeKey, find_spec, spec_registered = _sgl_registry.ShapeKey, _sgl_registry.find_spec, _sgl_registry.spec_registered
else:

    class Feature(enum.Enum):
        SPECULATIVE_DECODING = "speculative_decoding"
        PD_DISAGGREGATION = "pd_disaggregation"
        RAGGED_VERIFY = "ragged_verify"
        EAGLE3_HIDDEN_STATES = "eagle3_hidden_states"
        KV_OFFLOAD = "kv_offload"

    class NumericsKind(enum.Enum):
        TOLERANCE = "tolerance"
        EXACT = "exact"

    @dataclass(frozen=True)
    class Numerics:
        kind: NumericsKind
        bounds: dict = field(default_factory=dict)

        def bound(self, name: str) -> float:
            return self.bounds[name]

    @dataclass(frozen=True)
    class DeviceLimits:
        widths: tuple
        tp_sizes: tuple
        resident_blocks: int

    @dataclass(frozen=True)
    class Requirements:
        dtypes: frozenset = frozenset()
        attention_backends: frozenset = frozenset()
        server_args: dict = field(default_factory=dict)
        hf_config: dict = field(default_factory=dict)
        env: dict = field(default_factory=dict)

    @dataclass
    class MonoSpec:
        name: str
        devices: dict
        features: frozenset
        requires: Requirements
        numerics: Numerics
        model_disable_reasons: Callable[[Any, Any, dict], list]
        build: Callable[[Any, Any, Any], Any]
        api_version: int = 1
        config_disable_reasons: Callable[[Any, Any], list] | None = None
        load_tensor: Callable[[dict, Any, str, Any], None] | None = None
        unread_metadata: frozenset = frozenset()
        tokens_per_request: Callable[[Any], int] | None = None

        def widths(self, isa: str) -> tuple:
            return self.devices[isa].widths

    @dataclass(frozen=True)
    class ShapeKey:
        """The CUDA-graph key a step is routed by: identical on every rank, frozen at capture."""

        forward_mode: str  # "decode" | "target_verify"
        batch_size: int
        tokens_per_request: int = 1

        @property
        def rows(self) -> int:
            return self.batch_size * self.tokens_per_request

    _REGISTRY: dict = {}

    def register(*, backend: str, architecture: str, path: str, model_type: str | None = None) -> None:
        """Records "module:ATTR" under (backend, architecture, model_type); the module is
        imported only when a spec is looked up (``sgl_amd_mono/__init__.py:16-18``)."""
        _REGISTRY[(backend, architecture, model_type)] = path

    def _load(path: str):
        mod, attr = path.split(":")
        return getattr(importlib.import_module(mod), attr)

    def spec_registered(*, backend: str, architectures: list, model_type: str | None = None) -> bool:
        return any((backend, a, mt) in _REGISTRY for a in architectures for mt in (model_type, None))

    def find_spec(*, backend: str, architectures: list, isa: str, model_type: str | None = None):
        """(spec, "") or (None, why).  A spec registered for the model type wins over one
        registered for any model type (``test/unit/test_deepseek_v4_spec.py:41-62``)."""
        for arch in architectures:
            for mt in (model_type, None):
                path = _REGISTRY.get((backend, arch, mt))
                if path is None:
                    continue
                spec = _load(path)
                if isa not in spec.devices:
                    return None, f"{spec.name}: no kernels for {isa} (has {sorted(spec.devices)})"
                return spec, ""
        return None, f"no {backend} spec for {architectures} (model type {model_type!r})"


@dataclass
class Plan:
    """One routed step: the graph key and a per-step dict that the forward fills once
    (``glm53/spec.py:378,470,493``: ``plan.key``, ``plan.state``)."""

    key: "ShapeKey"
    state: dict = field(default_factory=dict)


@dataclass
class BuildContext:
    """What SGLang hands ``build`` (``glm53/spec.py:499-581``): the row counts its decode
    graphs will route, the wait deadline, and the dict every one-time copy is logged in."""

    widths: tuple
    deadline_s: float = 30.0
    copies: dict = field(default_factory=dict)
    tp_rank: int = 0
    tp_size: int = 1
    cpu_group: Any = None
    device: Any = "cuda:0"
    max_context: int = 16384
