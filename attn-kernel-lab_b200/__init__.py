"""B200-native (sm_100a) fused FP8 paged EXTEND/prefill attention.

Same consumer-facing names as the reference package (src/attn_kernel_lab/__init__.py):
the declared capability surface, the typed error that separates "outside the surface" from
a defect, and the operator entry points.  Import it as `attn_kernel_lab_b200` (the one-file module
of that name beside this directory loads it; the directory name itself is not an identifier).
"""
from .backend import BackendSettings, make_backend_class
from .capability import (
    CapabilityError,
    GENERALIZATION_CAPABILITY,
    KV_HEAD_SHARD_CAPABILITY,
    OperatorCapability,
    V1_CAPABILITY,
    check_supported,
)
from .kernel import NativeError, build, load, source_build_id
from .ops import (PrefillRequest, check_request, plan_batch_workspace, plan_workspace, prefill_extend,
                  prefill_extend_batch)
from .paged import fp8_paged_prefill
from .quant import (BatchPlan, CapacityPlan, FP8PrefillBatchWorkspace, FP8PrefillWorkspace,
                    WorkspaceCapacityError)

__all__ = [
    "CapabilityError", "GENERALIZATION_CAPABILITY", "KV_HEAD_SHARD_CAPABILITY", "OperatorCapability", "V1_CAPABILITY",
    "check_supported", "NativeError", "build", "load", "source_build_id", "PrefillRequest",
    "check_request", "plan_workspace", "plan_batch_workspace", "prefill_extend", "prefill_extend_batch",
    "CapacityPlan", "BatchPlan", "FP8PrefillBatchWorkspace",
    "FP8PrefillWorkspace", "WorkspaceCapacityError", "BackendSettings", "make_backend_class", "fp8_paged_prefill",
]

__version__ = "0.1.0"
