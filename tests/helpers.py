"""Shared helpers of the test-suite: plan conversion between the package and the oracle, tensors,
float comparison with the tolerances of the specification."""
import numpy as np

import attention_superoptimizer_b200 as mg
from oracle import mugraph_oracle as mo


def to_oracle_plan(plan: mg.ExecutionPlan) -> mo.ExecutionPlan:
    return mo.ExecutionPlan(ops=[(t, list(s)) for t, s in plan.ops], input_map=list(plan.input_map),
                            forloop_dim=list(plan.forloop_dim), input_smem_layouts=list(plan.input_smem_layouts),
                            output_map=tuple(plan.output_map), forloop_range=plan.forloop_range,
                            grid_dim=tuple(plan.grid_dim), block_dim=tuple(plan.block_dim),
                            reduction_dimx=plan.reduction_dimx)


def to_package_plan(plan: mo.ExecutionPlan) -> mg.ExecutionPlan:
    return mg.ExecutionPlan(ops=[(t, list(s)) for t, s in plan.ops], input_map=list(plan.input_map),
                            forloop_dim=list(plan.forloop_dim), input_smem_layouts=list(plan.input_smem_layouts),
                            output_map=tuple(plan.output_map), forloop_range=plan.forloop_range,
                            grid_dim=tuple(plan.grid_dim), block_dim=tuple(plan.block_dim),
                            reduction_dimx=plan.reduction_dimx)


def spec_of(t: mg.PyTensor) -> mo.DTensorSpec:
    return mo.DTensorSpec(tuple(t.shape), t.dtype, t.layout)


def f16_bits(x):
    return np.asarray(x, np.float32).astype(np.float16).view(np.uint16)


def bits_f16(b):
    return np.asarray(b, np.uint16).view(np.float16).astype(np.float32)


def bf16_bits(x):
    """round-to-nearest-even float32 -> bfloat16 bit patterns"""
    u = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r


def bits_bf16(b):
    return (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def to_bits(x, dtype):
    return f16_bits(x) if dtype == mg.float16 else bf16_bits(x)


def from_bits(b, dtype):
    return bits_f16(b) if dtype == mg.float16 else bits_bf16(b)


# Float-mode tolerance of the specification: 2e-3 relative for fp16, 1e-2 for bf16, against an fp32
# host evaluation.  "Relative" is taken against the magnitude of the tensor: an element may deviate by
# rtol * (|ref| + rms(ref)); the rms term keeps elements that cancel to ~0 from dominating.
RTOL = {mg.float16: 2e-3, mg.bfloat16: 1e-2}


def assert_close(got, ref, dtype, what="", outlier_fraction=0.0, outlier_cap=1.0):
    """Every element within rtol * (|ref| + rms(ref)).  `outlier_fraction` > 0 lets that share of the elements
    exceed the bound, but none by more than the factor `outlier_cap`: used only where the operand rounding of the
    16-bit tensor cores has a heavy tail of its own (un-normalised exp weights at full size, see the test that
    passes it).  Returns the worst relative error."""
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    rtol = RTOL[dtype]
    scale = np.sqrt(np.mean(ref ** 2)) + 1e-30
    rel = np.abs(got - ref) / (np.abs(ref) + scale)
    worst = float(np.max(rel))
    over = int(np.count_nonzero(rel > rtol))
    assert over <= outlier_fraction * rel.size, "%s: worst relative error %.3e > %.1e (%d elements over)" % (what, worst, rtol, over)
    assert worst <= rtol * max(1.0, outlier_cap), "%s: worst relative error %.3e > %.1e x %.2f" % (what, worst, rtol, outlier_cap)
    return worst
