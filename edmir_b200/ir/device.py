"""Device registry: static capabilities plus measured (calibrated) figures.

API and lookup behaviour follow the reference registry (EDM-IR/ir/device.py): ``DeviceSpec``
fields and derived properties (:69-140), fuzzy name matching where the longest alias wins
(:147-198), the built-in Hopper/Blackwell entries (:201-264), module-level helpers (:271-303)
and optional detection through torch or ``nvidia-smi`` (:306-371).

Two deliberate differences, both about sm_100: the reference marks every Blackwell part
``supports_wgmma=True`` (device.py:212-218), but wgmma exists on sm_90a only -- here the
Blackwell entries say ``False`` and carry ``attrs["tensor_core_isa"] = "tcgen05"``; and the
measured-bandwidth fields, which are ``None`` in every reference entry, can be filled for the
local B200 from a calibration table through ``install_calibration``.
"""
from __future__ import annotations

import re
import subprocess
from dataclasses import dataclass, field, replace
from typing import Any, Iterable

_NOISE_WORDS = ("nvidia", "geforce", "tesla", "gpu")


def _norm_name(name: str) -> str:
    text = name.lower()
    for word in _NOISE_WORDS:
        text = text.replace(word, "")
    return re.sub(r"[^a-z0-9]+", "", text)


def arch_from_compute_capability(cc: tuple[int, int] | None) -> str | None:
    if cc is None:
        return None
    return {9: "Hopper", 10: "Blackwell", 12: "Blackwell"}.get(cc[0])


@dataclass(frozen=True, slots=True)
class DeviceSpec:
    """What the analysis needs to know about a device: which mechanisms exist (static) and
    how fast the memory system and links were measured to be (calibrated, optional)."""

    name: str
    vendor: str = "NVIDIA"
    arch: str | None = None
    compute_capability: tuple[int, int] | None = None

    sm_count: int | None = None
    memory_bytes: int | None = None
    memory_kind: str | None = None
    memory_bandwidth_gbps: float | None = None

    supports_tensor_cores: bool = True
    supports_tma: bool = False
    supports_nvlink: bool = False
    supports_rdma: bool = False
    supports_wgmma: bool = False
    supports_fp8: bool = False

    nvlink_bandwidth_gbps: float | None = None
    pcie_bandwidth_gbps: float | None = None

    attrs: dict[str, Any] = field(default_factory=dict)

    @property
    def key(self) -> str:
        return _norm_name(self.name)

    @property
    def cuda_arch(self) -> str | None:
        if self.compute_capability is None:
            return None
        return "sm{}{}".format(*self.compute_capability)

    def _is_hbm(self) -> bool:
        return self.memory_kind is not None and self.memory_kind.upper().startswith("HBM")

    @property
    def hbm_bytes(self) -> int | None:
        return self.memory_bytes if self._is_hbm() else None

    @property
    def hbm_bandwidth_gbps(self) -> float | None:
        return self.memory_bandwidth_gbps if self._is_hbm() else None

    def with_runtime(self, *, name: str | None = None, sm_count: int | None = None,
                     memory_bytes: int | None = None, attrs: dict[str, Any] | None = None) -> "DeviceSpec":
        return replace(
            self,
            name=name or self.name,
            sm_count=self.sm_count if sm_count is None else sm_count,
            memory_bytes=self.memory_bytes if memory_bytes is None else memory_bytes,
            attrs={**self.attrs, **(attrs or {})},
        )


DeviceDesc = DeviceSpec  # older name kept for callers of earlier sketches


def _format_bytes(value: int | None) -> str:
    return "unknown" if value is None else f"{value / 2**30:.2f}GiB"


def format_device_spec(spec: DeviceSpec | None) -> str:
    if spec is None:
        return "device=<none>"
    parts = [
        f"name={spec.name}", f"vendor={spec.vendor}", f"arch={spec.arch}",
        f"cuda_arch={spec.cuda_arch}", f"cc={spec.compute_capability}",
        f"sm_count={spec.sm_count}", f"memory={_format_bytes(spec.memory_bytes)}",
        f"memory_kind={spec.memory_kind}",
    ]
    flags = (("tensor_cores", spec.supports_tensor_cores), ("tma", spec.supports_tma),
             ("wgmma", spec.supports_wgmma), ("fp8", spec.supports_fp8),
             ("nvlink", spec.supports_nvlink), ("rdma", spec.supports_rdma))
    on = [label for label, enabled in flags if enabled]
    if on:
        parts.append("features=" + ",".join(on))
    if spec.attrs:
        parts.append("attrs=" + ",".join(f"{k}={v}" for k, v in sorted(spec.attrs.items())))
    return "DeviceSpec(" + " ".join(parts) + ")"


class DeviceRegistry:
    """Specs by normalised name, plus loose aliases for profiler / runtime spellings."""

    def __init__(self) -> None:
        self._specs: dict[str, DeviceSpec] = {}
        self._aliases: dict[str, str] = {}

    def register(self, spec: DeviceSpec, *, aliases: Iterable[str] = (),
                 replace_existing: bool = False) -> DeviceSpec:
        key = spec.key
        if key in self._specs and not replace_existing:
            raise ValueError(f"device spec already registered: {spec.name}")
        self._specs[key] = spec
        for alias in (spec.name, *aliases):
            akey = _norm_name(alias)
            taken = self._aliases.get(akey)
            if taken is not None and taken != key and not replace_existing:
                raise ValueError(f"device alias already registered: {alias}")
            self._aliases[akey] = key
        return spec

    def match(self, raw_name: str) -> DeviceSpec | None:
        query = _norm_name(raw_name)
        direct = self._aliases.get(query)
        if direct is not None:
            return self._specs[direct]
        # runtime names carry memory sizes, SXM/PCIe suffixes, ...: try containment either
        # way round, longest alias first so "h200" is not shadowed by a shorter alias
        for alias in sorted(self._aliases, key=len, reverse=True):
            if alias and (alias in query or query in alias):
                return self._specs[self._aliases[alias]]
        return None

    def get(self, name: str) -> DeviceSpec:
        found = self.match(name)
        if found is None:
            raise KeyError(f"unknown device: {name}")
        return found

    def names(self) -> tuple[str, ...]:
        return tuple(s.name for s in self._specs.values())

    def specs(self) -> tuple[DeviceSpec, ...]:
        return tuple(self._specs.values())

    def supported(self) -> tuple[DeviceSpec, ...]:
        return tuple(s for s in self._specs.values() if s.arch in ("Hopper", "Blackwell"))


_BUILTINS = (
    # name, cc, memory kind, nvlink+rdma, aliases
    ("H100", (9, 0), "HBM", True, ("NVIDIA H100", "H100 PCIe", "H100 SXM", "H100 NVL", "sm90")),
    ("H200", (9, 0), "HBM", True, ("NVIDIA H200", "H200 SXM", "sm90 h200")),
    ("GH200", (9, 0), "HBM", True, ("NVIDIA GH200", "Grace Hopper", "GH200 Grace Hopper")),
    ("B200", (10, 0), "HBM", True, ("NVIDIA B200", "Blackwell B200", "sm100")),
    ("GB200", (10, 0), "HBM", True, ("NVIDIA GB200", "Grace Blackwell", "GB200 Grace Blackwell")),
    ("RTX 5090", (12, 0), "GDDR", False,
     ("NVIDIA GeForce RTX 5090", "GeForce RTX 5090", "RTX5090", "sm120")),
)


def _register_builtin_devices(registry: DeviceRegistry) -> None:
    for name, cc, mem, fabric, aliases in _BUILTINS:
        hopper = cc[0] == 9
        registry.register(
            DeviceSpec(
                name,
                arch=arch_from_compute_capability(cc),
                compute_capability=cc,
                memory_kind=mem,
                supports_tensor_cores=True,
                supports_tma=True,
                supports_nvlink=fabric,
                supports_rdma=fabric,
                supports_wgmma=hopper,  # wgmma is sm_90a only; sm_100 uses tcgen05
                supports_fp8=True,
                attrs={} if hopper else {"tensor_core_isa": "tcgen05" if cc[0] == 10 else "mma.sync"},
            ),
            aliases=aliases,
        )


DEFAULT_REGISTRY = DeviceRegistry()
_register_builtin_devices(DEFAULT_REGISTRY)


def register_device_spec(spec: DeviceSpec, *, aliases: Iterable[str] = (), replace_existing: bool = False,
                         registry: DeviceRegistry = DEFAULT_REGISTRY) -> DeviceSpec:
    return registry.register(spec, aliases=aliases, replace_existing=replace_existing)


def get_device_spec(name: str, *, registry: DeviceRegistry = DEFAULT_REGISTRY) -> DeviceSpec:
    return registry.get(name)


def match_device_spec(raw_name: str, *, registry: DeviceRegistry = DEFAULT_REGISTRY) -> DeviceSpec | None:
    return registry.match(raw_name)


def known_device_specs(*, registry: DeviceRegistry = DEFAULT_REGISTRY) -> tuple[DeviceSpec, ...]:
    return registry.specs()


def supported_nvidia_specs(*, registry: DeviceRegistry = DEFAULT_REGISTRY) -> tuple[DeviceSpec, ...]:
    return registry.supported()


def install_calibration(table: dict[str, Any], *, name: str = "B200",
                        registry: DeviceRegistry = DEFAULT_REGISTRY) -> DeviceSpec:
    """Fill the measured fields of a registered device from a calibration table
    (keys ``hbm_gbs``, ``nvlink_gbs_per_dir``, ``bf16_tflops``, anything else goes to ``attrs``)."""
    base = registry.get(name)
    extra = {k: v for k, v in table.items() if k not in ("hbm_gbs", "nvlink_gbs_per_dir")}
    spec = replace(
        base,
        memory_bandwidth_gbps=table.get("hbm_gbs", base.memory_bandwidth_gbps),
        nvlink_bandwidth_gbps=table.get("nvlink_gbs_per_dir", base.nvlink_bandwidth_gbps),
        attrs={**base.attrs, **extra},
    )
    return registry.register(spec, replace_existing=True)


# ---------------------------------------------------------------- detection (optional)
def detect_device(index: int = 0, *, registry: DeviceRegistry = DEFAULT_REGISTRY) -> DeviceSpec | None:
    """The local CUDA device as a spec, via torch if importable, else ``nvidia-smi``; ``None``
    when neither sees a GPU."""
    return _detect_with_torch(index, registry) or _detect_with_nvidia_smi(index, registry)


def _detect_with_torch(index: int, registry: DeviceRegistry) -> DeviceSpec | None:
    try:
        import torch

        if not torch.cuda.is_available():
            return None
        name = torch.cuda.get_device_name(index)
        props = torch.cuda.get_device_properties(index)
        cc = torch.cuda.get_device_capability(index)
    except Exception:
        return None
    base = registry.match(name)
    if base is None:
        modern = cc[0] >= 9
        base = DeviceSpec(name=name, arch=arch_from_compute_capability(cc), compute_capability=cc,
                          supports_tensor_cores=cc[0] >= 7, supports_tma=modern,
                          supports_wgmma=cc[0] == 9, supports_fp8=modern)
    return base.with_runtime(name=name, sm_count=getattr(props, "multi_processor_count", None),
                             memory_bytes=getattr(props, "total_memory", None),
                             attrs={"runtime": "torch", "cuda_index": index})


def _detect_with_nvidia_smi(index: int, registry: DeviceRegistry) -> DeviceSpec | None:
    cmd = ["nvidia-smi", f"--id={index}", "--query-gpu=name,memory.total", "--format=csv,noheader,nounits"]
    try:
        out = subprocess.run(cmd, check=True, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                             text=True, timeout=2.0).stdout.strip()
    except Exception:
        return None
    if not out:
        return None
    cells = [c.strip() for c in out.splitlines()[0].split(",")]
    mem = int(cells[1]) * 2**20 if len(cells) > 1 and cells[1].isdigit() else None
    base = registry.match(cells[0]) or DeviceSpec(name=cells[0])
    return base.with_runtime(name=cells[0], memory_bytes=mem,
                             attrs={"runtime": "nvidia-smi", "cuda_index": index})


__all__ = [
    "DEFAULT_REGISTRY", "DeviceDesc", "DeviceRegistry", "DeviceSpec",
    "arch_from_compute_capability", "detect_device", "format_device_spec", "get_device_spec",
    "install_calibration", "known_device_specs", "match_device_spec", "register_device_spec",
    "supported_nvidia_specs",
]
