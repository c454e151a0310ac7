"""saga_b200: B200-native fused gradient reduce-scatter + mixed-precision Adam +
weight all-gather, the data-parallel parameter update of the Saga framework,
behind a C ABI (include/b200opt.h, built into saga_b200/libb200opt.so).

The Python layer here is plumbing over that ABI: it mirrors the optimizer ops
and the step tail of Saga's CUDA backend so that tests and the benchmark can
drive the library the way Saga's program loop does.
"""
from . import capi, workload
from .optimizer import (AdamGroup, FlatLayout, LossScaler, TrainingStepTail,
                        policy_update, bias_corrections)

__all__ = ["capi", "workload", "AdamGroup", "FlatLayout", "LossScaler", "TrainingStepTail",
           "policy_update", "bias_corrections"]
