"""The ``.family`` and ``.task`` documents.

A FAMILY is the compile unit: one base scene and a constant slot table, hence constant state sizes for every task in
it.  A TASK is data: which slots are active, where each starts (a distribution, never a pose), what the goal is and what
the instruction says.  Both are ``key=value`` lines with repeating keys; an UNKNOWN KEY RAISES, because these files are
hand-written and every key is load-bearing (a dropped ``goal=`` is a task without a success condition).

    slot=<name>:<free|static>:<asset>[:x,y,z[,yaw]]          a static slot (no dofs) must carry its pose, a free one must not
    region=<name>:<site|box>:<site>[:xmin,ymin,xmax,ymax[:half_height[:<contact slot>]]]
    init=<slot>@<region or slot>[:in][:yaw][:sep=<metres>]   a slot name as the target stacks the object on that slot
    joint_init=<joint>:<lo>,<hi>
    goal=<predicate text>                                     carried as text; parsed by tasks/predicates.py

Reference: noeira/tasks/spec.mojo:50-1608.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import List, Optional

SCHEMA_VERSION = 1
SLOT_FREE, SLOT_STATIC = 0, 1
INIT_TARGET_REGION, INIT_TARGET_SLOT = 0, 1
STACK_Z_OFFSET = 0.01            # gap left under an object stacked on another object
TABLE_Z_OFFSET = 0.01            # gap left under an object placed on a table / floor region
DEFAULT_REGION_HALF_HEIGHT = 0.12
_SLOT_KINDS = {"free": SLOT_FREE, "static": SLOT_STATIC}


def _floats(text: str, what: str, n_min: int, n_max: int) -> List[float]:
    try:
        v = [float(x) for x in text.split(",")]
    except ValueError:
        raise ValueError(f"tasks: {what}: expected numbers, got {text!r}") from None
    if not n_min <= len(v) <= n_max:
        raise ValueError(f"tasks: {what}: expected {n_min}..{n_max} numbers, got {len(v)}")
    return v


def _num(x: float) -> str:
    return repr(float(x)) if float(x) != int(x) else str(int(x)) + ".0"


@dataclass
class SlotSpec:
    name: str
    kind: int
    asset: str
    pose: Optional[List[float]] = None      # x, y, z of a static slot
    yaw: float = 0.0                        # radians about +z
    bottom_z: float = 0.0                   # placement geometry read off the asset, when it declares it
    top_z: float = 0.0
    h_radius: float = 0.0
    has_geom: bool = False

    def set_geom(self, bottom_z: float, top_z: float, h_radius: float) -> None:
        self.bottom_z, self.top_z, self.h_radius, self.has_geom = bottom_z, top_z, h_radius, True

    def describe(self) -> str:
        s = f"{self.name}:{'static' if self.kind == SLOT_STATIC else 'free'}:{self.asset}"
        if self.pose is not None:
            s += ":" + ",".join(_num(x) for x in self.pose)
            if self.yaw != 0.0:
                s += "," + _num(self.yaw)
        return s


def parse_slot(text: str) -> SlotSpec:
    parts = text.split(":")
    if len(parts) not in (3, 4):
        raise ValueError(f"tasks: slot={text!r}: expected <name>:<kind>:<asset>[:x,y,z[,yaw]]")
    name, kind, asset = parts[0].strip(), parts[1].strip(), parts[2].strip()
    if kind not in _SLOT_KINDS:
        raise ValueError(f"tasks: unknown slot kind {kind!r} - expected 'free' (a movable prop, 6 dofs) or 'static' "
                         f"(a fixture, no dofs)")
    k = _SLOT_KINDS[kind]
    if k == SLOT_STATIC and len(parts) != 4:
        raise ValueError(f"tasks: static slot {name!r} needs a pose: it has no joint, so it cannot be moved after "
                         f"composition")
    if k == SLOT_FREE and len(parts) == 4:
        raise ValueError(f"tasks: free slot {name!r} must not carry a pose: its episode pose comes from the sampler")
    s = SlotSpec(name, k, asset)
    if len(parts) == 4:
        v = _floats(parts[3], f"slot {name}", 3, 4)
        s.pose, s.yaw = v[:3], (v[3] if len(v) == 4 else 0.0)
    return s


@dataclass
class RegionSpec:
    name: str
    site: str
    is_box: bool = False
    rect: Optional[List[float]] = None      # xmin, ymin, xmax, ymax relative to the site
    half_height: float = DEFAULT_REGION_HALF_HEIGHT
    has_height: bool = False
    contact: str = ""                       # box regions: optional contact partner slot

    def describe(self) -> str:
        s = f"{self.name}:{'box' if self.is_box else 'site'}:{self.site}"
        if self.rect is not None:
            s += ":" + ",".join(_num(x) for x in self.rect)
            if self.has_height:
                s += ":" + _num(self.half_height)
                if self.contact:
                    s += ":" + self.contact
        return s


def parse_region(text: str) -> RegionSpec:
    parts = [p.strip() for p in text.split(":")]
    if len(parts) < 3 or parts[1] not in ("site", "box"):
        raise ValueError(f"tasks: region={text!r}: expected <name>:<site|box>:<site>[:rect[:half_height[:contact]]]")
    r = RegionSpec(parts[0], parts[2], is_box=parts[1] == "box")
    if len(parts) > 3:
        r.rect = _floats(parts[3], f"region {r.name} rectangle", 4, 4)
        if r.rect[0] >= r.rect[2] or r.rect[1] >= r.rect[3]:
            raise ValueError(f"tasks: region {r.name}: empty rectangle {r.rect}")
    if len(parts) > 4:
        r.half_height, r.has_height = _floats(parts[4], f"region {r.name} half height", 1, 1)[0], True
        if r.half_height <= 0:
            raise ValueError(f"tasks: region {r.name}: half height must be positive")
    if len(parts) > 5:
        if not r.is_box:
            raise ValueError(f"tasks: region {r.name}: a contact partner belongs to a box region")
        r.contact = parts[5]
    if len(parts) > 6:
        raise ValueError(f"tasks: region={text!r}: too many fields")
    if r.is_box and (r.rect is None or not r.has_height):
        raise ValueError(f"tasks: box region {r.name} needs its rectangle and half height")
    return r


@dataclass
class InitSpec:
    slot: str
    region: str                 # a region name, or another slot's name (a stack)
    inside: bool = False        # ':in' - placed inside a fixture region, not on top of it
    yaw: bool = False           # ':yaw' - yaw drawn uniformly each episode
    sep_mm: int = 0             # ':sep=<metres>' - minimum centre distance to every other placed slot, whole millimetres

    def describe(self) -> str:
        s = f"{self.slot}@{self.region}"
        if self.inside:
            s += ":in"
        if self.yaw:
            s += ":yaw"
        if self.sep_mm:
            s += f":sep={self.sep_mm / 1000.0:g}"
        return s


def parse_init(text: str) -> InitSpec:
    head, *flags = [p.strip() for p in text.split(":")]
    if head.count("@") != 1:
        raise ValueError(f"tasks: init={text!r}: expected <slot>@<region or slot>")
    slot, target = (s.strip() for s in head.split("@"))
    if not slot or not target:
        raise ValueError(f"tasks: init={text!r}: empty slot or target")
    i = InitSpec(slot, target)
    for f in flags:
        if f == "in":
            i.inside = True
        elif f == "yaw":
            i.yaw = True
        elif f.startswith("sep="):
            mm = round(_floats(f[4:], f"init {slot} sep", 1, 1)[0] * 1000.0)
            if not 1 <= mm <= 1023:
                raise ValueError(f"tasks: init {slot}: sep must be 0.001 .. 1.023 m")
            i.sep_mm = int(mm)
        else:
            raise ValueError(f"tasks: init={text!r}: unknown flag {f!r} (known: in, yaw, sep=<metres>)")
    return i


@dataclass
class JointInitSpec:
    joint: str
    lo: float
    hi: float

    def describe(self) -> str:
        return f"{self.joint}:{_num(self.lo)},{_num(self.hi)}"


def parse_joint_init(text: str) -> JointInitSpec:
    if text.count(":") != 1:
        raise ValueError(f"tasks: joint_init={text!r}: expected <joint>:<lo>,<hi>")
    j, rng = (s.strip() for s in text.split(":"))
    lo, hi = _floats(rng, f"joint_init {j}", 2, 2)
    if lo > hi:
        raise ValueError(f"tasks: joint_init {j}: lo > hi")
    return JointInitSpec(j, lo, hi)


def _kv_lines(text: str, what: str):
    for ln, raw in enumerate(text.splitlines(), 1):
        line = raw.strip()
        if not line or line.startswith("#"):
            continue
        if "=" not in line:
            raise ValueError(f"tasks: {what}:{ln}: expected key=value, got {raw!r}")
        k, v = line.split("=", 1)
        yield ln, k.strip(), v.strip()


def _check_version(v: str, what: str) -> int:
    if int(v) != SCHEMA_VERSION:
        raise ValueError(f"tasks: {what}: schema_version {v} is not readable by this build (reads {SCHEMA_VERSION})")
    return int(v)


@dataclass
class FamilySpec:
    name: str = ""
    base: str = ""
    horizon: int = 200
    control_freq: int = 20
    slots: List[SlotSpec] = field(default_factory=list)
    regions: List[RegionSpec] = field(default_factory=list)
    park: List[float] = field(default_factory=lambda: [10.0, 0.0, 50.0])   # where inactive free slots wait
    base_pos: List[float] = field(default_factory=lambda: [0.0, 0.0, 0.0])
    floor: bool = True
    root: str = ""

    def slot_index(self, name: str) -> int:
        for i, s in enumerate(self.slots):
            if s.name == name:
                return i
        raise KeyError(f"tasks: family {self.name!r} has no slot {name!r} (slots: {[s.name for s in self.slots]})")

    def region_index(self, name: str) -> int:
        for i, r in enumerate(self.regions):
            if r.name == name:
                return i
        raise KeyError(f"tasks: family {self.name!r} has no region {name!r} (regions: {[r.name for r in self.regions]})")

    def has_slot(self, name: str) -> bool:
        return any(s.name == name for s in self.slots)

    def has_region(self, name: str) -> bool:
        return any(r.name == name for r in self.regions)

    def init_target_kind(self, name: str) -> int:
        """The one resolver of an ``init=`` / ``On`` target: a region or a slot, never both."""
        r, s = self.has_region(name), self.has_slot(name)
        if r and s:
            raise ValueError(f"tasks: {name!r} names both a region and a slot of family {self.name!r}")
        if not r and not s:
            raise KeyError(f"tasks: {name!r} is neither a region nor a slot of family {self.name!r}")
        return INIT_TARGET_REGION if r else INIT_TARGET_SLOT

    def to_text(self) -> str:
        out = [f"schema_version={SCHEMA_VERSION}", f"name={self.name}", f"base={self.base}", f"horizon={self.horizon}",
               f"control_freq={self.control_freq}", "park=" + ",".join(_num(x) for x in self.park),
               "base_pos=" + ",".join(_num(x) for x in self.base_pos), f"floor={'1' if self.floor else '0'}"]
        out += [f"slot={s.describe()}" for s in self.slots]
        out += [f"region={r.describe()}" for r in self.regions]
        return "\n".join(out) + "\n"


_FAMILY_KEYS = "schema_version, name, base, horizon, control_freq, park, base_pos, floor, slot, region"


def parse_family(text: str, what: str = "<family>") -> FamilySpec:
    f = FamilySpec()
    seen_version = False
    for ln, k, v in _kv_lines(text, what):
        if k == "schema_version":
            _check_version(v, what)
            seen_version = True
        elif k == "name":
            f.name = v
        elif k == "base":
            f.base = v
        elif k == "horizon":
            f.horizon = int(v)
        elif k == "control_freq":
            f.control_freq = int(v)
        elif k == "park":
            f.park = _floats(v, "park", 3, 3)
        elif k == "base_pos":
            f.base_pos = _floats(v, "base_pos", 3, 3)
        elif k == "floor":
            if v not in ("0", "1"):
                raise ValueError(f"tasks: {what}:{ln}: floor must be 0 or 1")
            f.floor = v == "1"
        elif k == "slot":
            f.slots.append(parse_slot(v))
        elif k == "region":
            f.regions.append(parse_region(v))
        else:
            raise ValueError(f"tasks: {what}:{ln}: unknown key {k!r}. Known: {_FAMILY_KEYS}")
    if not seen_version:
        raise ValueError(f"tasks: {what}: missing schema_version=")
    if not f.name:
        raise ValueError(f"tasks: {what}: missing name=")
    names = [s.name for s in f.slots]
    if len(set(names)) != len(names):
        raise ValueError(f"tasks: {what}: duplicate slot names")
    rn = [r.name for r in f.regions]
    if len(set(rn)) != len(rn):
        raise ValueError(f"tasks: {what}: duplicate region names")
    for r in f.regions:
        if r.contact and not f.has_slot(r.contact):
            raise ValueError(f"tasks: {what}: region {r.name}: contact partner {r.contact!r} is not a slot")
    return f


@dataclass
class TaskSpec:
    name: str = ""
    family: str = ""
    suite: str = ""
    language: str = ""
    active: List[str] = field(default_factory=list)
    inits: List[InitSpec] = field(default_factory=list)
    joint_inits: List[JointInitSpec] = field(default_factory=list)
    goal: str = ""
    horizon: int = 0            # 0 = the family's

    def to_text(self) -> str:
        out = [f"schema_version={SCHEMA_VERSION}", f"name={self.name}", f"family={self.family}"]
        if self.suite:
            out.append(f"suite={self.suite}")
        out.append(f"language={self.language}")
        if self.horizon:
            out.append(f"horizon={self.horizon}")
        out += [f"active={a}" for a in self.active]
        out += [f"init={i.describe()}" for i in self.inits]
        out += [f"joint_init={j.describe()}" for j in self.joint_inits]
        out.append(f"goal={self.goal}")
        return "\n".join(out) + "\n"


_TASK_KEYS = "schema_version, name, family, suite, language, horizon, active, init, joint_init, goal"


def parse_task(text: str, what: str = "<task>") -> TaskSpec:
    t = TaskSpec()
    seen_version = False
    for ln, k, v in _kv_lines(text, what):
        if k == "schema_version":
            _check_version(v, what)
            seen_version = True
        elif k == "name":
            t.name = v
        elif k == "family":
            t.family = v
        elif k == "suite":
            t.suite = v
        elif k == "language":
            t.language = v
        elif k == "horizon":
            t.horizon = int(v)
        elif k == "active":
            t.active.append(v)
        elif k == "init":
            t.inits.append(parse_init(v))
        elif k == "joint_init":
            t.joint_inits.append(parse_joint_init(v))
        elif k == "goal":
            if t.goal:
                raise ValueError(f"tasks: {what}:{ln}: a task has ONE goal; combine terms with And(...)")
            t.goal = v
        else:
            raise ValueError(f"tasks: {what}:{ln}: unknown key {k!r}. Known: {_TASK_KEYS}")
    if not seen_version:
        raise ValueError(f"tasks: {what}: missing schema_version=")
    if not t.name or not t.family:
        raise ValueError(f"tasks: {what}: missing name= or family=")
    if not t.goal:
        raise ValueError(f"tasks: {what}: missing goal= (a task without a success condition)")
    return t


def order_inits(t: TaskSpec, f: FamilySpec) -> List[InitSpec]:
    """Placement order: region draws first, then stacks, each after the slot it stands on."""
    done, out = set(), []
    pending = list(t.inits)
    while pending:
        progressed = False
        for i in list(pending):
            kind = f.init_target_kind(i.region)
            if kind == INIT_TARGET_REGION or i.region in done:
                out.append(i)
                done.add(i.slot)
                pending.remove(i)
                progressed = True
        if not progressed:
            raise ValueError(f"tasks: task {t.name!r}: stack cycle or a stack on an unplaced slot among "
                             f"{[i.describe() for i in pending]}")
    return out


def validate_task_against_family(t: TaskSpec, f: FamilySpec) -> None:
    if t.family != f.name:
        raise ValueError(f"tasks: task {t.name!r} belongs to family {t.family!r}, not {f.name!r}")
    for a in t.active:
        f.slot_index(a)
    if len(set(t.active)) != len(t.active):
        raise ValueError(f"tasks: task {t.name!r}: a slot is activated twice")
    placed = set()
    for i in t.inits:
        s = f.slots[f.slot_index(i.slot)]
        if i.slot not in t.active:
            raise ValueError(f"tasks: task {t.name!r}: init for {i.slot!r}, which is not active")
        if s.kind == SLOT_STATIC:
            raise ValueError(f"tasks: task {t.name!r}: {i.slot!r} is static; it cannot be placed")
        if i.slot in placed:
            raise ValueError(f"tasks: task {t.name!r}: two inits for {i.slot!r}")
        placed.add(i.slot)
        kind = f.init_target_kind(i.region)
        if kind == INIT_TARGET_SLOT:
            if i.region not in t.active:
                raise ValueError(f"tasks: task {t.name!r}: {i.slot!r} is stacked on inactive slot {i.region!r}")
            if i.yaw:
                raise ValueError(f"tasks: task {t.name!r}: a stacked init takes no :yaw (there is no draw)")
    for a in t.active:
        if f.slots[f.slot_index(a)].kind == SLOT_FREE and a not in placed:
            raise ValueError(f"tasks: task {t.name!r}: active free slot {a!r} has no init= (it would stay parked)")
    order_inits(t, f)


def load_family(path: str) -> FamilySpec:
    with open(path, "r", encoding="utf-8") as fh:
        f = parse_family(fh.read(), path)
    f.root = os.path.dirname(os.path.dirname(os.path.abspath(path)))
    return f


def load_task(path: str) -> TaskSpec:
    with open(path, "r", encoding="utf-8") as fh:
        return parse_task(fh.read(), path)
