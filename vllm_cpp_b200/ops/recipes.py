"""Fusion-recipe catalogue: what each fused producer computes, as data.

A recipe is a short list of row-wise steps over named values. Each recipe can be realised three
ways, and the three must agree:

  tier 2  the bespoke kernel written for it (``bespoke``), when there is one;
  tier 1  the fused-chain interpreter (``csrc/kernels/recipe.cu``): ONE launch for any recipe made
          of row steps, the intermediate rows in shared memory;
  tier 0  the composite: one plain kernel per step (or, with ``backend="torch"``, the fp32 PyTorch
          restatement, which is what the CPU tests and the numerics oracle use).

Tier 1 reproduces the bytes of the GPU composite (same rounding points, same summation order);
bespoke kernels that reduce in another order may differ from it in the last bf16 bit of a
normalised value, and the GPU tests bound that.

``run(recipe, tensors)`` picks the highest tier available, so a model can ask for a fusion by
name and get one launch whether or not a hand-written kernel exists for it.

Reference: include/vt/recipes.h:38-352 (the constexpr recipe table), include/vt/fused_recipe.h
(step / operand encoding), src/vt/cuda/cuda_ops.cu:1238 (the interpreter kernel).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

ACTS = {"silu": 0, "gelu_tanh": 1, "gelu_erf": 2}
GATES = {"silu": 0, "sigmoid": 1}

# interpreter opcodes (csrc/kernels/recipe.cu)
OP_LOAD, OP_STORE, OP_ADD, OP_RMSNORM, OP_RMSNORM_GATED, OP_ACT_MUL, OP_SIGMOID_MUL, OP_QUANT_FP8, \
    OP_QUANT_NVFP4 = range(9)
MAX_STEPS, MAX_OPERANDS, MAX_REGS = 16, 12, 4


@dataclass(frozen=True)
class Step:
    """``out = op(a, b; params)``. ``a`` / ``b`` / ``out`` name row values; ``w`` / ``scale`` name
    vector or scalar operands; ``attrs`` holds compile-time choices (activation kind, gemma)."""
    op: str
    out: str
    a: str
    b: Optional[str] = None
    w: Optional[str] = None
    scale: Optional[str] = None
    attrs: tuple = ()

    def attr(self, key, default=None):
        return dict(self.attrs).get(key, default)


@dataclass(frozen=True)
class FusedRecipe:
    name: str
    inputs: tuple            # row tensors read from memory: bf16 [T, heads * width]
    params: tuple            # vector / scalar operands and python scalars (eps)
    steps: tuple
    outputs: tuple           # values written back, in order
    inplace: tuple = ()      # (value, input) pairs: the value is stored over that input tensor
    per_head: bool = False   # rows are heads of width w.numel() inside wider token rows
    interpretable: bool = True
    bespoke: Optional[str] = None     # name in _BESPOKE
    reference: str = ""


def _s(op, out, a, b=None, w=None, scale=None, **attrs):
    return Step(op, out, a, b, w, scale, tuple(sorted(attrs.items())))


CATALOG: dict[str, FusedRecipe] = {}


def _register(r: FusedRecipe) -> FusedRecipe:
    CATALOG[r.name] = r
    return r


FUSED_ADD_RMSNORM = _register(FusedRecipe(
    "fused_add_rmsnorm_gemma", ("x", "residual"), ("w", "eps"),
    (_s("add", "h", "x", "residual"), _s("rmsnorm", "y", "h", w="w", gemma=True)),
    ("y", "h"), inplace=(("h", "residual"),), bespoke="add_rmsnorm",
    reference="include/vt/recipes.h kFusedAddRmsNorm"))
FUSED_ADD_RMSNORM_STD = _register(FusedRecipe(
    "fused_add_rmsnorm", ("x", "residual"), ("w", "eps"),
    (_s("add", "h", "x", "residual"), _s("rmsnorm", "y", "h", w="w", gemma=False)),
    ("y", "h"), inplace=(("h", "residual"),), bespoke="add_rmsnorm",
    reference="include/vt/recipes.h kFusedAddRmsNormStd"))
RMSNORM_QUANT_FP8 = _register(FusedRecipe(
    "rmsnorm_quant_fp8", ("x",), ("w", "eps", "scale"),
    (_s("rmsnorm", "y", "x", w="w", gemma=False), _s("quant_fp8", "q", "y", scale="scale")),
    ("q",), bespoke="rmsnorm_quant_fp8", reference="include/vt/recipes.h kRmsNormQuantFp8"))
RMSNORM_GATED_QUANT_FP8 = _register(FusedRecipe(
    "rmsnorm_gated_quant_fp8", ("x", "z"), ("w", "eps", "scale"),
    (_s("rmsnorm_gated", "y", "x", "z", w="w", gate="silu"), _s("quant_fp8", "q", "y", scale="scale")),
    ("q",), per_head=True, reference="include/vt/recipes.h kRmsNormGatedQuantFp8"))
SILU_MUL_QUANT_NVFP4 = _register(FusedRecipe(
    "silu_mul_quant_nvfp4", ("gate", "up"), ("gscale",),
    (_s("act_mul", "y", "gate", "up", act="silu"), _s("quant_nvfp4", "q", "y", scale="gscale")),
    ("q",), bespoke="silu_mul_quant_nvfp4", reference="include/vt/recipes.h kSiluMulFp4Quant"))
SILU_MUL_QUANT_FP8 = _register(FusedRecipe(
    "silu_mul_quant_fp8", ("gate", "up"), ("scale",),
    (_s("act_mul", "y", "gate", "up", act="silu"), _s("quant_fp8", "q", "y", scale="scale")),
    ("q",), reference="include/vt/recipes.h kSiluMulQuantFp8"))
SIGMOID_GATE_QUANT_NVFP4 = _register(FusedRecipe(
    "sigmoid_gate_quant_nvfp4", ("x", "gate"), ("gscale",),
    (_s("sigmoid_mul", "y", "x", "gate"), _s("quant_nvfp4", "q", "y", scale="gscale")),
    ("q",), bespoke="sigmoid_gate_quant_nvfp4", reference="include/vt/recipes.h kSigmoidGateFp4Quant"))
ADD_RMSNORM_QUANT_NVFP4 = _register(FusedRecipe(
    "add_rmsnorm_quant_nvfp4", ("x", "residual"), ("w", "eps", "gscale"),
    (_s("add", "h", "x", "residual"), _s("rmsnorm", "y", "h", w="w", gemma=False),
     _s("quant_nvfp4", "q", "y", scale="gscale")),
    ("q", "h"), inplace=(("h", "residual"),), bespoke="add_rmsnorm_quant_nvfp4",
    reference="(no counterpart: the W4A4 input of a layer's first projection)"))
# Per-head q/k RMSNorm + rotary embedding (+ the split of an interleaved q|gate projection) are one
# kernel together with the KV-cache write (ops.rope_kv); their steps address heads and positions,
# which the row interpreter does not, so they exist as the bespoke kernel and the PyTorch composite.
ATTN_QK_NORM_ROPE = _register(FusedRecipe(
    "attn_qk_norm_rope", ("qkv",), ("q_norm", "k_norm", "eps", "positions", "cos_sin"),
    (_s("head_rmsnorm", "qn", "qkv", w="q_norm", gemma=True), _s("rope", "q", "qn", w="cos_sin"),
     _s("head_rmsnorm", "kn", "qkv", w="k_norm", gemma=True), _s("rope", "k", "kn", w="cos_sin")),
    ("q", "k"), per_head=True, interpretable=False, bespoke="rope_kv",
    reference="include/vt/recipes.h kAttnQkNormRope"))
ATTN_QK_NORM_ROPE_GATE = _register(FusedRecipe(
    "attn_qk_norm_rope_gate", ("qkv",), ("q_norm", "k_norm", "eps", "positions", "cos_sin"),
    (_s("split_gate", "qg", "qkv"), _s("head_rmsnorm", "qn", "qg", w="q_norm", gemma=True),
     _s("rope", "q", "qn", w="cos_sin"),
     _s("head_rmsnorm", "kn", "qkv", w="k_norm", gemma=True), _s("rope", "k", "kn", w="cos_sin")),
    ("q", "k"), per_head=True, interpretable=False, bespoke="rope_kv",
    reference="include/vt/recipes.h kAttnQkNormRopeGate; src/vt/cuda/cuda_ops.cu:964"))


# ---------------------------------------------------------------------------------------------
# tier 0: the composite
# ---------------------------------------------------------------------------------------------
def _heads_of(recipe, t, w):
    return t.shape[1] // w.numel() if recipe.per_head else 1


def _torch_step(st: Step, env, recipe):
    a = env[st.a].float()
    bf = lambda v: v.to(torch.bfloat16)
    if st.op == "add":
        return bf(a + env[st.b].float())
    if st.op == "rmsnorm":
        w = env[st.w].float() + (1.0 if st.attr("gemma") else 0.0)
        return bf(a * torch.rsqrt((a * a).mean(-1, keepdim=True) + env["eps"]) * w)
    if st.op == "rmsnorm_gated":
        w = env[st.w]
        T, heads = a.shape[0], _heads_of(recipe, a, w)
        x = a.reshape(T, heads, -1)
        z = env[st.b].float().reshape(T, heads, -1)
        g = torch.nn.functional.silu(z) if st.attr("gate", "silu") == "silu" else torch.sigmoid(z)
        return bf((x * torch.rsqrt((x * x).mean(-1, keepdim=True) + env["eps"]) * w.float() * g).reshape(T, -1))
    if st.op == "act_mul":
        kind = st.attr("act", "silu")
        act = {"silu": torch.nn.functional.silu,
               "gelu_tanh": lambda v: torch.nn.functional.gelu(v, approximate="tanh"),
               "gelu_erf": torch.nn.functional.gelu}[kind]
        return bf(act(a) * env[st.b].float())
    if st.op == "sigmoid_mul":
        return bf(a * torch.sigmoid(env[st.b].float()))
    if st.op == "quant_fp8":
        return (a / env[st.scale].float()).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    if st.op == "quant_nvfp4":
        from .quant import ref_quant_nvfp4_activations
        return ref_quant_nvfp4_activations(env[st.a], env[st.scale])
    raise NotImplementedError(f"step '{st.op}' has no composite")


def _gpu_step(st: Step, env, recipe):
    from .. import ops
    from . import gdn as G, quant as Q
    a = env[st.a]
    if st.op == "add":
        return ops.add(a, env[st.b])
    if st.op == "rmsnorm":
        return ops.rmsnorm(a, env[st.w], env["eps"], gemma=bool(st.attr("gemma")))
    if st.op == "rmsnorm_gated":
        w = env[st.w]
        return G.rmsnorm_gated(a, env[st.b], w, torch.empty_like(a), env["eps"], st.attr("gate", "silu"),
                               heads=_heads_of(recipe, a, w))
    if st.op == "act_mul":
        return ops.act_and_mul(torch.cat([a, env[st.b]], dim=1), ACTS[st.attr("act", "silu")])
    if st.op == "sigmoid_mul":
        return ops.sigmoid_mul(a, env[st.b])
    if st.op == "quant_fp8":
        return Q.quant_fp8(a, env[st.scale])
    if st.op == "quant_nvfp4":
        return Q.quant_nvfp4(a, env[st.scale], swizzle=bool(env.get("swizzle", False)))
    raise NotImplementedError(f"step '{st.op}' has no composite")


def run_composite(recipe: FusedRecipe, tensors: dict, backend: str = "gpu") -> dict:
    """One kernel (``backend="gpu"``) or one PyTorch expression (``"torch"``) per step. Returns
    {output name: tensor}; in-place outputs are also copied over their input tensor."""
    if not all(st.op in _COMPOSITE_OPS for st in recipe.steps):
        raise NotImplementedError(f"recipe '{recipe.name}' is realised by its bespoke kernel only")
    env = dict(tensors)
    step = _gpu_step if backend == "gpu" else _torch_step
    for st in recipe.steps:
        env[st.out] = step(st, env, recipe)
    for val, inp in recipe.inplace:
        tensors[inp].copy_(env[val])
    return {o: env[o] for o in recipe.outputs}


_COMPOSITE_OPS = {"add", "rmsnorm", "rmsnorm_gated", "act_mul", "sigmoid_mul", "quant_fp8", "quant_nvfp4"}


# ---------------------------------------------------------------------------------------------
# tier 1: the interpreter
# ---------------------------------------------------------------------------------------------
class B200ChainStep(ctypes.Structure):
    _fields_ = [("op", ctypes.c_int), ("dst", ctypes.c_int), ("a", ctypes.c_int), ("b", ctypes.c_int),
                ("operand", ctypes.c_int), ("operand2", ctypes.c_int), ("operand3", ctypes.c_int),
                ("flag", ctypes.c_int), ("f", ctypes.c_float)]


class B200ChainOperand(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("ld", ctypes.c_longlong), ("col", ctypes.c_longlong)]


class B200Chain(ctypes.Structure):
    _fields_ = [("n_steps", ctypes.c_int), ("n_regs", ctypes.c_int), ("width", ctypes.c_int),
                ("heads", ctypes.c_int), ("rows", ctypes.c_longlong),
                ("steps", B200ChainStep * MAX_STEPS), ("operands", B200ChainOperand * MAX_OPERANDS)]


@dataclass
class ChainPlan:
    """A recipe lowered to interpreter steps: register numbers assigned, operand slots named."""
    steps: list = field(default_factory=list)      # (op, dst, a, b, operand, operand2, operand3, flag, f-name)
    operands: list = field(default_factory=list)   # operand names, slot order
    n_regs: int = 0


def lower(recipe: FusedRecipe) -> ChainPlan:
    """Loads before first use, stores after the producing step, registers reused once a value is
    dead (a recipe needs at most MAX_REGS live rows)."""
    if not recipe.interpretable:
        raise NotImplementedError(f"recipe '{recipe.name}' is not a chain of row steps")
    plan = ChainPlan()
    last_use: dict[str, int] = {}
    for i, st in enumerate(recipe.steps):
        for v in (st.a, st.b):
            if v is not None:
                last_use[v] = i
    stored = dict((val, inp) for val, inp in recipe.inplace)
    reg_of: dict[str, int] = {}
    free = list(range(MAX_REGS))

    def slot(name):
        if name not in plan.operands:
            plan.operands.append(name)
        return plan.operands.index(name)

    def alloc(name):
        if not free:
            raise NotImplementedError(f"recipe '{recipe.name}' needs more than {MAX_REGS} live rows")
        reg_of[name] = free.pop(0)
        plan.n_regs = max(plan.n_regs, reg_of[name] + 1)
        return reg_of[name]

    for i, st in enumerate(recipe.steps):
        for v in (st.a, st.b):
            if v is not None and v not in reg_of:
                if v not in recipe.inputs:
                    raise ValueError(f"recipe '{recipe.name}': '{v}' is used before it is made")
                plan.steps.append((OP_LOAD, alloc(v), 0, 0, slot(v), 0, 0, 0, None))
        a = reg_of[st.a]
        b = reg_of[st.b] if st.b is not None else 0
        # values that die at this step free their registers before the result is placed, so an
        # element-wise step may write over its own input
        for v in sorted({st.a, st.b} - {None}):
            if last_use.get(v) == i:            # (an output was stored when it was made)
                free.insert(0, reg_of[v])
        if st.op in ("quant_fp8", "quant_nvfp4"):
            if st.op == "quant_fp8":
                plan.steps.append((OP_QUANT_FP8, 0, a, 0, slot(st.out), slot(st.scale), 0, 0, None))
            else:
                plan.steps.append((OP_QUANT_NVFP4, 0, a, 0, slot(st.out), slot(st.out + ".sf"), slot(st.scale),
                                   "swizzle", None))
            continue
        dst = alloc(st.out)
        if st.op == "add":
            plan.steps.append((OP_ADD, dst, a, b, 0, 0, 0, 0, None))
        elif st.op == "rmsnorm":
            plan.steps.append((OP_RMSNORM, dst, a, 0, slot(st.w), 0, 0, int(bool(st.attr("gemma"))), "eps"))
        elif st.op == "rmsnorm_gated":
            plan.steps.append((OP_RMSNORM_GATED, dst, a, b, slot(st.w), 0, 0, GATES[st.attr("gate", "silu")], "eps"))
        elif st.op == "act_mul":
            plan.steps.append((OP_ACT_MUL, dst, a, b, 0, 0, 0, ACTS[st.attr("act", "silu")], None))
        elif st.op == "sigmoid_mul":
            plan.steps.append((OP_SIGMOID_MUL, dst, a, b, 0, 0, 0, 0, None))
        else:
            raise NotImplementedError(f"step '{st.op}' is not a row step")
        if st.out in recipe.outputs:
            plan.steps.append((OP_STORE, 0, dst, 0, slot(stored.get(st.out, st.out)), 0, 0, 0, None))
        if st.out not in last_use and st.out in reg_of:
            free.insert(0, reg_of[st.out])       # stored and never read again
    if len(plan.steps) > MAX_STEPS or len(plan.operands) > MAX_OPERANDS:
        raise NotImplementedError(f"recipe '{recipe.name}' is too long for one chain")
    return plan


_PLANS: dict[str, ChainPlan] = {}
_declared = False


def _declare():
    global _declared
    if not _declared:
        from . import _lib
        _lib.declare("b200_fused_chain", [ctypes.POINTER(B200Chain), _lib.P], _lib.I)
        _declared = True


def _alloc_outputs(recipe, tensors, T, K, device, swizzle):
    """Output tensors the caller did not pass: bf16 rows, fp8 rows, or the NVFP4 (packed, scales) pair."""
    made = {}
    inplace = dict(recipe.inplace)
    for st in recipe.steps:
        if st.out not in recipe.outputs or st.out in inplace:
            continue
        if st.op == "quant_fp8":
            made[st.out] = tensors.get(st.out)
            if made[st.out] is None:
                made[st.out] = torch.empty((T, K), dtype=torch.float8_e4m3fn, device=device)
        elif st.op == "quant_nvfp4":
            pair = tensors.get(st.out)
            if pair is None:
                n_sf = ((T + 127) // 128) * 128 * (K // 16) if swizzle else T * (K // 16)
                pair = (torch.empty((T, K // 2), dtype=torch.uint8, device=device),
                        torch.zeros(n_sf, dtype=torch.uint8, device=device))
            made[st.out] = pair
        else:
            made[st.out] = tensors.get(st.out)
            if made[st.out] is None:
                made[st.out] = torch.empty((T, K), dtype=torch.bfloat16, device=device)
    return made


def run_interpreter(recipe: FusedRecipe, tensors: dict) -> dict:
    """The whole recipe as one launch of the fused-chain kernel."""
    from . import _lib
    from ._lib import check, lib, ptr, stream_ptr
    _declare()
    plan = _PLANS.get(recipe.name)
    if plan is None:
        plan = _PLANS[recipe.name] = lower(recipe)
    first = tensors[recipe.inputs[0]]
    T, K = first.shape
    heads = 1
    if recipe.per_head:
        w = next(tensors[st.w] for st in recipe.steps if st.w is not None)
        heads = K // w.numel()
    width = K // heads
    swizzle = bool(tensors.get("swizzle", False))
    outs = _alloc_outputs(recipe, tensors, T, K, first.device, swizzle)
    prog = B200Chain()
    prog.n_steps, prog.n_regs, prog.width, prog.heads, prog.rows = len(plan.steps), plan.n_regs, width, heads, T * heads
    for i, name in enumerate(plan.operands):
        if name.endswith(".sf"):
            t = outs[name[:-3]][1]
        elif name in outs:
            t = outs[name][0] if isinstance(outs[name], tuple) else outs[name]
        else:
            t = tensors[name]
        if t.dim() == 2 and t.stride(1) != 1:
            raise ValueError(f"operand '{name}' must have unit column stride")
        prog.operands[i].ptr = ptr(t)
        prog.operands[i].ld = t.stride(0) if t.dim() == 2 and name not in recipe.params else 0
        prog.operands[i].col = 0
    for i, (op, dst, a, b, o1, o2, o3, flag, fname) in enumerate(plan.steps):
        s = prog.steps[i]
        s.op, s.dst, s.a, s.b, s.operand, s.operand2, s.operand3 = op, dst, a, b, o1, o2, o3
        s.flag = int(swizzle) if flag == "swizzle" else flag
        s.f = float(tensors[fname]) if fname else 0.0
    check(lib().b200_fused_chain(ctypes.byref(prog), stream_ptr()), f"fused_chain[{recipe.name}]")
    res = {}
    inplace = dict(recipe.inplace)
    for o in recipe.outputs:
        res[o] = tensors[inplace[o]] if o in inplace else outs[o]
        if isinstance(res[o], tuple) and not swizzle:
            res[o] = (res[o][0], res[o][1].view(T, K // 16))     # row-major scales, as the quantiser returns them
    return res


# ---------------------------------------------------------------------------------------------
# tier 2: bespoke kernels
# ---------------------------------------------------------------------------------------------
def _b_add_rmsnorm(recipe, t):
    from .. import ops
    gemma = bool(recipe.steps[1].attr("gemma"))
    y = ops.rmsnorm(t["x"], t["w"], t["eps"], residual=t["residual"], gemma=gemma, out=t.get("y"))
    return {"y": y, "h": t["residual"]}


def _b_rmsnorm_quant_fp8(recipe, t):
    from . import quant as Q
    return {"q": Q.quant_fp8(t["x"], t["scale"], out=t.get("q"), norm_weight=t["w"], eps=t["eps"])}


def _b_silu_mul_quant_nvfp4(recipe, t):
    from . import quant as Q
    gate, up = t["gate"], t["up"]
    # the kernel reads [gate | up] rows; two views of one merged projection output pass straight through
    if (gate.data_ptr() + gate.shape[1] * 2 == up.data_ptr()) and gate.stride(0) == up.stride(0):
        gu = torch.as_strided(gate, (gate.shape[0], 2 * gate.shape[1]), (gate.stride(0), 1))
    else:
        gu = torch.cat([gate, up], dim=1)
    return {"q": Q.quant_nvfp4(gu, t["gscale"], silu_mul=True, swizzle=bool(t.get("swizzle", False)), out=t.get("q"))}


def _b_sigmoid_gate_quant_nvfp4(recipe, t):
    from . import quant as Q
    return {"q": Q.quant_nvfp4_gated(t["x"], t["gate"], t["gscale"], swizzle=bool(t.get("swizzle", False)),
                                     out=t.get("q"))}


def _b_add_rmsnorm_quant_nvfp4(recipe, t):
    from . import quant as Q
    q = Q.rmsnorm_quant_nvfp4(t["x"], t["w"], t["eps"], t["gscale"], residual=t["residual"],
                              swizzle=bool(t.get("swizzle", False)), out=t.get("q"))
    return {"q": q, "h": t["residual"]}


_BESPOKE: dict[str, Callable] = {
    "add_rmsnorm": _b_add_rmsnorm,
    "rmsnorm_quant_fp8": _b_rmsnorm_quant_fp8,
    "silu_mul_quant_nvfp4": _b_silu_mul_quant_nvfp4,
    "sigmoid_gate_quant_nvfp4": _b_sigmoid_gate_quant_nvfp4,
    "add_rmsnorm_quant_nvfp4": _b_add_rmsnorm_quant_nvfp4,
    "rope_kv": None,       # called by the attention layers with their cache arguments (ops.rope_kv)
}


def tiers(recipe: FusedRecipe) -> tuple:
    """Which realisations exist, best first."""
    out = []
    if recipe.bespoke:
        out.append("bespoke")
    if recipe.interpretable:
        out.append("interpreter")
    if all(st.op in _COMPOSITE_OPS for st in recipe.steps):
        out.append("composite")
    return tuple(out)


def run(recipe: FusedRecipe | str, tensors: dict, tier: str | None = None) -> dict:
    """Run a recipe on GPU tensors. ``tensors`` maps the recipe's inputs and params (plus optional
    pre-allocated outputs and ``swizzle`` for NVFP4 scale layout) to tensors / scalars. ``tier``:
    "bespoke", "interpreter", "composite", or None for the best one there is. CPU tensors run the
    PyTorch composite."""
    if isinstance(recipe, str):
        recipe = CATALOG[recipe]
    first = tensors[recipe.inputs[0]]
    if first.device.type != "cuda":
        return run_composite(recipe, tensors, backend="torch")
    tier = tier or tiers(recipe)[0]
    if tier == "bespoke":
        fn = _BESPOKE.get(recipe.bespoke)
        if fn is None:
            raise NotImplementedError(f"recipe '{recipe.name}' is called through its layer, not by name")
        return fn(recipe, tensors)
    if tier == "interpreter":
        return run_interpreter(recipe, tensors)
    return run_composite(recipe, tensors, backend="gpu")


def describe() -> list:
    """One row per recipe: name, steps, tiers, reference: what ``tools dump-ops`` prints."""
    return [{"name": r.name, "steps": [s.op for s in r.steps], "tiers": list(tiers(r)), "reference": r.reference}
            for r in CATALOG.values()]
