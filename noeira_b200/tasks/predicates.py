"""The goal language: ``goal=In(brick, box_inside)``.

Two passes, and the split is the design:

    parse_goal("And(In(brick, box_inside), Upright(brick))")  -> a tree of terms holding NAMES
    bind_goal(tree, family, joints)                            -> a postfix TAPE of (op, a, b, param) holding INDICES

The tape is what runs where the reward runs: ``evaluate`` (tensor program, any device) and the CUDA kernel
``goal_eval_kernel`` (csrc/tasks.cu, one thread per environment, a bit stack) read the same four arrays, so success
and the shaping distance cost no host round trip per step.  Strings are resolved once, at task-load time.

Predicates (positions are slot origins; a region is a rectangle and a vertical band about its site):
    In(obj, region)        inside the rectangle and |z - site z| <= the region's half height
    AtRegion(obj, region)  the same test; reads better for an end effector
    On(obj, region)        inside the rectangle and the object's bottom 0 .. 3 cm above the site
    On(obj, obj2)          bound to ON_BODY: centres within 3 cm in xy and the bottom of obj -1 .. +3 cm from obj2's top
    Near(a, b, d)          centre distance below d
    Above(a, b, margin)    z_a - z_b > margin  (the margin is why a brick resting on a table is not "above" it)
    Upright(obj[, c])      the body's z axis within acos(c) of world z (default c = 0.9)
    Joint(joint, cmp, thr) qpos[joint] <cmp> thr, cmp in lt / le / gt / ge
    And(...), Or(...), Not(x)
    Touching, Grasped      parse and bind, but need contact data the batched state does not carry: refused by
                           ``require_evaluable`` (and by the tape), never silently approximated.
The op codes are the wire format of the device tape: append, never renumber.
Reference: noeira/tasks/predicates.mojo:1-687, noeira/tasks/eval.mojo (semantics of the tests).
"""
from __future__ import annotations

import ctypes
import re
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .spec import INIT_TARGET_REGION, FamilySpec

OP_IN, OP_ON, OP_NEAR, OP_ABOVE, OP_UPRIGHT, OP_OPEN, OP_AT_REGION, OP_TOUCHING, OP_GRASPED = range(9)
OP_AND, OP_OR, OP_NOT, OP_JOINT, OP_ON_BODY = 9, 10, 11, 12, 13
OP_COUNT = 14
CMP_LT, CMP_LE, CMP_GT, CMP_GE = 0, 1, 2, 3
_CMP = {"lt": CMP_LT, "le": CMP_LE, "gt": CMP_GT, "ge": CMP_GE}
_NAMES = {"In": OP_IN, "On": OP_ON, "Near": OP_NEAR, "Above": OP_ABOVE, "Upright": OP_UPRIGHT, "Open": OP_OPEN,
          "AtRegion": OP_AT_REGION, "Touching": OP_TOUCHING, "Grasped": OP_GRASPED, "And": OP_AND, "Or": OP_OR,
          "Not": OP_NOT, "Joint": OP_JOINT}
_ARITY = {OP_IN: (2, 2), OP_ON: (2, 2), OP_NEAR: (3, 3), OP_ABOVE: (3, 3), OP_UPRIGHT: (1, 2), OP_OPEN: (1, 1),
          OP_AT_REGION: (2, 2), OP_TOUCHING: (2, 2), OP_GRASPED: (1, 1), OP_JOINT: (3, 3)}
ON_BAND = 0.03          # an object "on" a surface has its bottom at most this far above it
ON_BODY_XY = 0.03       # and, on another object, its centre this close in xy
ON_BODY_BELOW = 0.01
MAX_TERMS = 32          # capacity of the device tape (and of the kernel's bit stack)


@dataclass
class Term:
    op: int
    args: List[str] = field(default_factory=list)        # names / numbers of a leaf
    children: List["Term"] = field(default_factory=list)  # And / Or / Not

    def describe(self) -> str:
        name = next(k for k, v in _NAMES.items() if v == self.op)
        inner = ", ".join(c.describe() for c in self.children) if self.children else ", ".join(self.args)
        return f"{name}({inner})"


def _split_args(s: str) -> List[str]:
    out, depth, cur = [], 0, ""
    for ch in s:
        if ch == "(":
            depth += 1
        elif ch == ")":
            depth -= 1
            if depth < 0:
                raise ValueError("tasks: goal: unbalanced ')'")
        if ch == "," and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if depth != 0:
        raise ValueError("tasks: goal: unbalanced '('")
    if cur.strip():
        out.append(cur.strip())
    return out


def parse_goal(text: str) -> Term:
    text = text.strip()
    m = re.fullmatch(r"([A-Za-z]+)\((.*)\)", text, re.S)
    if not m:
        raise ValueError(f"tasks: goal {text!r}: expected Name(args)")
    name, inner = m.group(1), m.group(2)
    if name not in _NAMES:
        raise ValueError(f"tasks: goal: unknown predicate {name!r}. Known: {sorted(_NAMES)}")
    op = _NAMES[name]
    args = _split_args(inner)
    if op in (OP_AND, OP_OR):
        if len(args) < 2:
            raise ValueError(f"tasks: goal: {name} needs at least two terms")
        return Term(op, children=[parse_goal(a) for a in args])
    if op == OP_NOT:
        if len(args) != 1:
            raise ValueError("tasks: goal: Not takes one term")
        return Term(op, children=[parse_goal(args[0])])
    lo, hi = _ARITY[op]
    if not lo <= len(args) <= hi:
        raise ValueError(f"tasks: goal: {name} takes {lo}{'' if lo == hi else '..' + str(hi)} arguments, got {len(args)}")
    return Term(op, args=args)


@dataclass
class BoundGoal:
    """Postfix tape: term i is (op[i], a[i], b[i], param[i]); And / Or carry their operand count in ``a``."""
    op: List[int] = field(default_factory=list)
    a: List[int] = field(default_factory=list)
    b: List[int] = field(default_factory=list)
    param: List[float] = field(default_factory=list)

    def __len__(self):
        return len(self.op)

    def push(self, op, a=0, b=0, param=0.0):
        if len(self.op) >= MAX_TERMS:
            raise ValueError(f"tasks: goal has more than {MAX_TERMS} terms")
        self.op.append(int(op)); self.a.append(int(a)); self.b.append(int(b)); self.param.append(float(param))

    def tensors(self, device):
        return (torch.tensor(self.op, dtype=torch.int32, device=device), torch.tensor(self.a, dtype=torch.int32, device=device),
                torch.tensor(self.b, dtype=torch.int32, device=device), torch.tensor(self.param, dtype=torch.float32, device=device))


def _number(s: str, what: str) -> float:
    try:
        return float(s)
    except ValueError:
        raise ValueError(f"tasks: goal: {what}: expected a number, got {s!r}") from None


def bind_goal(goal: Term, family: FamilySpec, joints: Optional[Dict[str, int]] = None) -> BoundGoal:
    """Resolves every name once.  ``joints`` maps a joint name to its qpos address."""
    bg = BoundGoal()

    def emit(t: Term):
        if t.op in (OP_AND, OP_OR):
            for c in t.children:
                emit(c)
            bg.push(t.op, a=len(t.children))
        elif t.op == OP_NOT:
            emit(t.children[0])
            bg.push(OP_NOT)
        elif t.op in (OP_IN, OP_AT_REGION):
            bg.push(t.op, family.slot_index(t.args[0]), family.region_index(t.args[1]))
        elif t.op == OP_ON:
            subj = family.slot_index(t.args[0])
            if family.init_target_kind(t.args[1]) == INIT_TARGET_REGION:
                bg.push(OP_ON, subj, family.region_index(t.args[1]), ON_BAND)
            else:
                bg.push(OP_ON_BODY, subj, family.slot_index(t.args[1]), ON_BODY_XY)
        elif t.op == OP_NEAR:
            bg.push(OP_NEAR, family.slot_index(t.args[0]), family.slot_index(t.args[1]), _number(t.args[2], "Near distance"))
        elif t.op == OP_ABOVE:
            bg.push(OP_ABOVE, family.slot_index(t.args[0]), family.slot_index(t.args[1]), _number(t.args[2], "Above margin"))
        elif t.op == OP_UPRIGHT:
            bg.push(OP_UPRIGHT, family.slot_index(t.args[0]), 0, _number(t.args[1], "Upright cosine") if len(t.args) > 1 else 0.9)
        elif t.op == OP_JOINT:
            if joints is None or t.args[0] not in joints:
                raise KeyError(f"tasks: goal: unknown joint {t.args[0]!r}")
            if t.args[1] not in _CMP:
                raise ValueError(f"tasks: unknown comparison {t.args[1]!r}. Known: lt, le, gt, ge.")
            bg.push(OP_JOINT, joints[t.args[0]], _CMP[t.args[1]], _number(t.args[2], "Joint threshold"))
        elif t.op == OP_TOUCHING:
            bg.push(OP_TOUCHING, family.slot_index(t.args[0]), family.slot_index(t.args[1]))
        elif t.op in (OP_GRASPED, OP_OPEN):
            bg.push(t.op, family.slot_index(t.args[0]))
        else:
            raise ValueError(f"tasks: goal: cannot bind op {t.op}")

    emit(goal)
    return bg


def require_evaluable(bg: BoundGoal) -> None:
    for op in bg.op:
        if op in (OP_TOUCHING, OP_GRASPED, OP_OPEN):
            name = next(k for k, v in _NAMES.items() if v == op)
            raise ValueError(f"tasks: goal uses {name}, which needs contact / grasp data the batched state does not carry")


@dataclass
class GoalState:
    """What the predicates read, batched over N environments."""
    pos: torch.Tensor            # [N, S, 3] slot origins
    quat: torch.Tensor           # [N, S, 4] (w, x, y, z)
    site: torch.Tensor           # [N, R, 3] region site positions
    rect: torch.Tensor           # [R, 5]   xmin, ymin, xmax, ymax, half_height
    geom: torch.Tensor           # [S, 3]   bottom_z, top_z, h_radius of every slot's asset
    qpos: Optional[torch.Tensor] = None   # [N, nq]


def family_tables(family: FamilySpec, device) -> tuple:
    """(rect [R,5], geom [S,3]) of a family; a region without a rectangle gets a 1 cm square about its site."""
    rect = torch.tensor([[*(r.rect if r.rect is not None else (-0.01, -0.01, 0.01, 0.01)), r.half_height]
                         for r in family.regions] or [[0, 0, 0, 0, 0]], dtype=torch.float32, device=device)
    geom = torch.tensor([[s.bottom_z, s.top_z, s.h_radius] for s in family.slots] or [[0, 0, 0]], dtype=torch.float32,
                        device=device)
    return rect, geom


def _leaf(op, a, b, prm, st: GoalState):
    """→ (satisfied [N] bool, distance to satisfaction [N] float >= 0)."""
    if op in (OP_IN, OP_AT_REGION, OP_ON):
        d = st.pos[:, a] - st.site[:, b]
        r = st.rect[b]
        ox = torch.clamp(r[0] - d[:, 0], min=0) + torch.clamp(d[:, 0] - r[2], min=0)
        oy = torch.clamp(r[1] - d[:, 1], min=0) + torch.clamp(d[:, 1] - r[3], min=0)
        if op == OP_ON:
            h = d[:, 2] + st.geom[a, 0]               # bottom of the object above the site
            oz = torch.clamp(-h, min=0) + torch.clamp(h - prm, min=0)
        else:
            oz = torch.clamp(d[:, 2].abs() - r[4], min=0)
        dist = ox + oy + oz
        return dist <= 0, dist
    if op == OP_ON_BODY:
        d = st.pos[:, a] - st.pos[:, b]
        dxy = torch.clamp(torch.linalg.vector_norm(d[:, :2], dim=-1) - prm, min=0)
        h = d[:, 2] + st.geom[a, 0] - st.geom[b, 1]   # bottom of a above the top of b
        dz = torch.clamp(-ON_BODY_BELOW - h, min=0) + torch.clamp(h - ON_BAND, min=0)
        dist = dxy + dz
        return dist <= 0, dist
    if op == OP_NEAR:
        dist = torch.clamp(torch.linalg.vector_norm(st.pos[:, a] - st.pos[:, b], dim=-1) - prm, min=0)
        return dist <= 0, dist
    if op == OP_ABOVE:
        g = st.pos[:, a, 2] - st.pos[:, b, 2] - prm
        return g > 0, torch.clamp(-g, min=0)
    if op == OP_UPRIGHT:
        q = st.quat[:, a]
        zz = 1.0 - 2.0 * (q[:, 1] * q[:, 1] + q[:, 2] * q[:, 2])   # world-z component of the body's z axis
        return zz >= prm, torch.clamp(prm - zz, min=0)
    if op == OP_JOINT:
        v = st.qpos[:, a]
        if b == CMP_LT:
            return v < prm, torch.clamp(v - prm, min=0)
        if b == CMP_LE:
            return v <= prm, torch.clamp(v - prm, min=0)
        if b == CMP_GT:
            return v > prm, torch.clamp(prm - v, min=0)
        return v >= prm, torch.clamp(prm - v, min=0)
    raise ValueError(f"tasks: op {op} is not evaluable")


def evaluate(bg: BoundGoal, st: GoalState):
    """Tensor-program evaluation of the tape → (success [N] bool, distance [N] float).  The distance of And is the
    sum of its terms', of Or the minimum, of Not 0 / 1; it is the shaping potential (0 exactly when satisfied for
    Not-free goals)."""
    require_evaluable(bg)
    stack = []
    for op, a, b, prm in zip(bg.op, bg.a, bg.b, bg.param):
        if op == OP_AND or op == OP_OR:
            terms = [stack.pop() for _ in range(a)]
            s = terms[0][0]
            d = terms[0][1]
            for ts, td in terms[1:]:
                s = (s & ts) if op == OP_AND else (s | ts)
                d = (d + td) if op == OP_AND else torch.minimum(d, td)
            stack.append((s, d))
        elif op == OP_NOT:
            s, _ = stack.pop()
            stack.append((~s, s.float()))
        else:
            stack.append(_leaf(op, a, b, prm, st))
    assert len(stack) == 1, "malformed goal tape"
    return stack[0]


def evaluate_cuda(bg: BoundGoal, st: GoalState, tape=None):
    """The same through ``goal_eval_kernel`` (one thread per environment).  ``tape``: cached ``bg.tensors(device)``."""
    from .._native import check, cuda_lib, ptr, stream_ptr
    require_evaluable(bg)
    dev = st.pos.device
    op, a, b, prm = tape if tape is not None else bg.tensors(dev)
    N, S, R = st.pos.shape[0], st.pos.shape[1], st.site.shape[1]
    ok = torch.empty(N, dtype=torch.uint8, device=dev)
    dist = torch.empty(N, dtype=torch.float32, device=dev)
    qpos = st.qpos if st.qpos is not None else torch.zeros(N, 1, device=dev)
    c = ctypes
    check(cuda_lib().nb_goal_eval(ptr(st.pos.contiguous()), ptr(st.quat.contiguous()), ptr(st.site.contiguous()),
                                  ptr(st.rect.contiguous()), ptr(st.geom.contiguous()), ptr(qpos.contiguous()),
                                  c.c_int(N), c.c_int(S), c.c_int(R), c.c_int(qpos.shape[1]), ptr(op), ptr(a), ptr(b), ptr(prm),
                                  c.c_int(len(bg)), ptr(ok), ptr(dist), stream_ptr()), "goal_eval")
    return ok.bool(), dist
