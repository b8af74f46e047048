"""EDM-IR node, graph, analysis and device API (same public names as the reference package,
EDM-IR/ir/__init__.py:38-70), re-implemented for the B200 backend."""
from .analysis import (
    CriticalPathResult,
    ExposureResult,
    OverlapGainResult,
    analyze_critical_path,
    analyze_exposure,
    analyze_overlap,
)
from .builder import EDMBuilder
from .device import (
    DEFAULT_REGISTRY,
    DeviceDesc,
    DeviceRegistry,
    DeviceSpec,
    arch_from_compute_capability,
    detect_device,
    format_device_spec,
    get_device_spec,
    known_device_specs,
    match_device_spec,
    register_device_spec,
    supported_nvidia_specs,
)
from .graph import EDMGraph, Edge
from .uop import (
    DATA_BUFFER,
    DATA_CONST,
    DATA_PARAM,
    DataRef,
    MovementDesc,
    TensorDesc,
    UOp,
    buffer_ref,
    const_ref,
    param_ref,
)

__all__ = sorted(
    name for name, value in list(globals().items())
    if not name.startswith("_") and not isinstance(value, type(__import__("sys")))
)
