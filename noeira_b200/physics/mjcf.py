"""MJCF subset → ``RigidModel``.

Supported: ``<compiler angle="degree|radian" coordinate="local">``, ``<option timestep gravity>``, nested ``<default>``
classes (``class`` / ``childclass`` resolution for ``joint``, ``geom``, ``motor``), ``<include file>`` relative to the
including file, ``<worldbody>`` with nested ``<body pos quat euler axisangle>``, ``<joint type="hinge|slide" axis pos
range damping armature stiffness springref ref>``, ``<geom type="capsule|sphere" size fromto pos quat rgba friction
density contype>``, explicit ``<inertial pos mass diaginertia>``, ``<actuator><motor joint gear ctrlrange>``.
World-level ``<geom type="plane">`` sets the ground plane.  Anything else raises ``MjcfError`` naming the element,
so an unsupported model never loads silently wrong.  (The reference's parser covers the whole schema,
noeira/physics3d/parser/; the env zoo here only needs trees of hinge / slide joints with capsule and sphere geoms.)
"""
from __future__ import annotations

import copy
import os
import xml.etree.ElementTree as ET
from typing import Dict, List, Optional

import numpy as np

from .model import (HINGE, SLIDE, Actuator, Body, Geom, Joint, Options, RigidModel, quat_from_axis_angle, quat_mul,
                    quat_z_to)


class MjcfError(ValueError):
    pass


def _floats(s, n=None):
    v = [float(x) for x in s.replace(",", " ").split()]
    if n is not None and len(v) != n:
        raise MjcfError(f"expected {n} numbers, got {s!r}")
    return v


class _Defaults:
    """Default classes: ``defaults[cls][tag]`` = attribute dict, children inherit from their parent class."""

    def __init__(self):
        self.cls: Dict[str, Dict[str, Dict[str, str]]] = {"main": {}}

    def load(self, elem, parent="main"):
        name = elem.get("class", parent if elem.get("class") is None and parent == "main" else None) or "main"
        base = copy.deepcopy(self.cls.get(parent, {}))
        for ch in elem:
            if ch.tag == "default":
                continue
            base.setdefault(ch.tag, {}).update(ch.attrib)
        self.cls[name] = base
        for ch in elem:
            if ch.tag == "default":
                self.load(ch, name)

    def resolve(self, tag, elem, childclass):
        cls = elem.get("class") or childclass or "main"
        if cls not in self.cls:
            raise MjcfError(f"unknown default class {cls!r}")
        out = dict(self.cls[cls].get(tag, {}))
        out.update(elem.attrib)
        return out


def _expand_includes(root, base_dir):
    for parent in list(root.iter()):
        for i, ch in enumerate(list(parent)):
            if ch.tag == "include":
                path = os.path.join(base_dir, ch.get("file"))
                sub = ET.parse(path).getroot()
                _expand_includes(sub, os.path.dirname(path))
                parent.remove(ch)
                for k, g in enumerate(list(sub) if sub.tag in ("mujoco", "mujocoinclude") else [sub]):
                    parent.insert(i + k, g)


def _quat_of(attrs, degrees):
    if "quat" in attrs:
        return np.array(_floats(attrs["quat"], 4))
    if "axisangle" in attrs:
        a = _floats(attrs["axisangle"], 4)
        return quat_from_axis_angle(a[:3], np.deg2rad(a[3]) if degrees else a[3])
    if "euler" in attrs:
        e = _floats(attrs["euler"], 3)
        if degrees:
            e = [np.deg2rad(x) for x in e]
        q = np.array([1.0, 0, 0, 0])
        for ax, ang in zip(((1, 0, 0), (0, 1, 0), (0, 0, 1)), e):      # intrinsic xyz
            q = quat_mul(q, quat_from_axis_angle(ax, ang))
        return q
    return np.array([1.0, 0, 0, 0])


def from_mjcf(source: str, opt: Optional[Options] = None, general: bool = False):
    """``source``: a file path or an XML string.  By default the result is a ``RigidModel`` for the fused step (hinge / slide
    trees, capsule / sphere geoms); ``general=True`` also accepts free and ball joints (``<freejoint/>``, ``type="free"`` /
    ``"ball"``) and box geoms and returns a ``physics.general.GeneralModel``."""
    if source.lstrip().startswith("<"):
        root, base_dir = ET.fromstring(source), "."
    else:
        root, base_dir = ET.parse(source).getroot(), os.path.dirname(os.path.abspath(source))
    if root.tag != "mujoco":
        raise MjcfError(f"root element is <{root.tag}>, expected <mujoco>")
    _expand_includes(root, base_dir)
    degrees = True
    for c in root.findall("compiler"):
        degrees = c.get("angle", "degree") == "degree"
        if c.get("coordinate", "local") != "local":
            raise MjcfError("only coordinate=\"local\" is supported")
    o = opt or Options()
    for e in root.findall("option"):
        if "timestep" in e.attrib:
            o.timestep = float(e.get("timestep"))
        if "gravity" in e.attrib:
            o.gravity = tuple(_floats(e.get("gravity"), 3))
    defaults = _Defaults()
    for d in root.findall("default"):
        defaults.load(d)
    wb = root.find("worldbody")
    if wb is None:
        raise MjcfError("no <worldbody>")
    bodies: List[Body] = []
    has_plane = False
    # assets with their data inline: <mesh name vertex="x y z …" scale="…"/> (the convex hull of the points is the shape) and
    # <hfield name nrow ncol size="rx ry top base" elevation="…"/> (values in [0, 1] scaled by ``top``); file references raise
    meshes, hfields = {}, {}
    for asset in root.findall("asset"):
        for e in asset:
            if e.tag == "mesh":
                if "vertex" not in e.attrib:
                    raise MjcfError(f"mesh {e.get('name')!r}: only inline vertex=\"…\" data is supported, not files")
                v = np.array(_floats(e.get("vertex"))).reshape(-1, 3) * np.array(_floats(e.get("scale", "1 1 1"), 3))
                meshes[e.get("name")] = [tuple(float(x) for x in r) for r in v]
            elif e.tag == "hfield":
                if "elevation" not in e.attrib:
                    raise MjcfError(f"hfield {e.get('name')!r}: only inline elevation=\"…\" data is supported, not files")
                nrow, ncol = int(e.get("nrow")), int(e.get("ncol"))
                rx, ry, top, _base = _floats(e.get("size"), 4)
                hfields[e.get("name")] = (np.array(_floats(e.get("elevation"), nrow * ncol)).reshape(nrow, ncol) * top, rx, ry)
    hfield = None

    def ang(x):
        return np.deg2rad(x) if degrees else x

    def parse_geom(a) -> Optional[Geom]:
        typ = a.get("type", "sphere")
        size = _floats(a.get("size", "0"))
        rgba = tuple(_floats(a.get("rgba", "0.7 0.7 0.7 1"), 4))
        fr = _floats(a.get("friction", "1"))[0]
        dens = float(a.get("density", "1000"))
        contact = a.get("contype", "1") != "0" or a.get("conaffinity", "1") != "0"
        if typ == "capsule":
            if "fromto" in a:
                ft = np.array(_floats(a["fromto"], 6))
                p0, p1 = ft[:3], ft[3:]
                return Geom("capsule", (size[0], 0.5 * float(np.linalg.norm(p1 - p0))), tuple(0.5 * (p0 + p1)),
                            tuple(quat_z_to(p1 - p0)), fr, dens, rgba, contact)
            if len(size) < 2:
                raise MjcfError("capsule needs size=\"radius half_length\" or fromto")
            return Geom("capsule", (size[0], size[1]), tuple(_floats(a.get("pos", "0 0 0"), 3)), tuple(_quat_of(a, degrees)),
                        fr, dens, rgba, contact)
        if typ == "sphere":
            return Geom("sphere", (size[0],), tuple(_floats(a.get("pos", "0 0 0"), 3)), (1.0, 0, 0, 0), fr, dens, rgba, contact)
        if typ == "box" and general:
            return Geom("box", tuple(size[:3]), tuple(_floats(a.get("pos", "0 0 0"), 3)), tuple(_quat_of(a, degrees)), fr, dens, rgba,
                        contact)
        if typ == "mesh" and general:
            name = a.get("mesh")
            if name not in meshes:
                raise MjcfError(f"geom refers to mesh {name!r}, which <asset> does not define with inline vertices")
            return Geom("mesh", (float(a.get("margin", "0")),), tuple(_floats(a.get("pos", "0 0 0"), 3)), tuple(_quat_of(a, degrees)),
                        fr, dens, rgba, contact, vertices=meshes[name])
        raise MjcfError(f"geom type {typ!r} is not supported (capsule, sphere; box and mesh in the general engine; plane and "
                        "hfield at world level)")

    def parse_body(elem, parent, childclass):
        cc = elem.get("childclass", childclass)
        joints, geoms = [], []
        mass = inertia = ipos = None
        for ch in elem:
            if ch.tag == "joint":
                a = defaults.resolve("joint", ch, cc)
                jt = a.get("type", "hinge")
                if jt in ("free", "ball") and general:
                    from .general import BALL, FREE
                    joints.append(Joint(FREE if jt == "free" else BALL, (0.0, 0.0, 1.0), tuple(_floats(a.get("pos", "0 0 0"), 3)),
                                        name=a.get("name", f"joint{len(bodies)}_{len(joints)}")))
                    continue
                if jt not in ("hinge", "slide"):
                    raise MjcfError(f"joint type {jt!r} is not supported (hinge, slide; free / ball in the general engine)")
                rng = None
                if "range" in a and a.get("limited", "auto") != "false":
                    r = _floats(a["range"], 2)
                    rng = tuple(ang(x) for x in r) if jt == "hinge" else tuple(r)
                ref = float(a.get("ref", "0"))
                joints.append(Joint(HINGE if jt == "hinge" else SLIDE, tuple(_floats(a.get("axis", "0 0 1"), 3)),
                                    tuple(_floats(a.get("pos", "0 0 0"), 3)), rng, float(a.get("armature", "0")),
                                    float(a.get("damping", "0")), float(a.get("stiffness", "0")),
                                    ang(float(a.get("springref", "0"))) if jt == "hinge" else float(a.get("springref", "0")),
                                    ang(ref) if jt == "hinge" else ref, a.get("name", f"joint{len(bodies)}_{len(joints)}")))
            elif ch.tag == "geom":
                geoms.append(parse_geom(defaults.resolve("geom", ch, cc)))
            elif ch.tag == "inertial":
                mass = float(ch.get("mass"))
                ipos = tuple(_floats(ch.get("pos", "0 0 0"), 3))
                if "diaginertia" in ch.attrib:
                    inertia = tuple(_floats(ch.get("diaginertia"), 3))
            elif ch.tag == "freejoint":
                if not general:
                    raise MjcfError("free / ball joints are not supported by the fused step (nq == nv trees only): general=True")
                from .general import FREE
                joints.append(Joint(FREE, (0.0, 0.0, 1.0), name=ch.get("name", f"joint{len(bodies)}_{len(joints)}")))
            elif ch.tag not in ("body", "site", "camera", "light"):
                raise MjcfError(f"<{ch.tag}> inside <body> is not supported")
        idx = len(bodies)
        bodies.append(Body(parent, tuple(_floats(elem.get("pos", "0 0 0"), 3)), tuple(_quat_of(elem.attrib, degrees)), joints, geoms,
                           elem.get("name", f"body{idx}"), mass, inertia, ipos))
        for ch in elem:
            if ch.tag == "body":
                parse_body(ch, idx, cc)

    for ch in wb:
        if ch.tag == "body":
            parse_body(ch, -1, None)
        elif ch.tag == "geom":
            a = defaults.resolve("geom", ch, None)
            if a.get("type", "sphere") == "hfield" and general:
                from .narrowphase import HeightField
                if a.get("hfield") not in hfields:
                    raise MjcfError(f"geom refers to hfield {a.get('hfield')!r}, which <asset> does not define inline")
                data, rx, ry = hfields[a["hfield"]]
                hfield = HeightField(data, rx, ry, tuple(_floats(a.get("pos", "0 0 0"), 3)), _floats(a.get("friction", "1"))[0])
                continue
            if a.get("type", "sphere") != "plane":
                raise MjcfError("world-level geoms other than the ground plane (and a height field in the general engine) are not supported")
            p = _floats(a.get("pos", "0 0 0"), 3)
            o.plane_offset = p[2]
            has_plane = True
        elif ch.tag not in ("light", "camera", "site"):
            raise MjcfError(f"<{ch.tag}> in <worldbody> is not supported")
    if not bodies:
        raise MjcfError("no bodies")
    acts = []
    for act in root.findall("actuator"):
        for m in act:
            if m.tag not in ("motor", "general"):
                raise MjcfError(f"actuator <{m.tag}> is not supported (motor)")
            a = defaults.resolve("motor", m, None)
            acts.append(Actuator(a["joint"], _floats(a.get("gear", "1"))[0], tuple(_floats(a.get("ctrlrange", "-1 1"), 2))))
    if general:
        from .general import GeneralModel, Motor
        return GeneralModel(bodies, [Motor(a.joint, a.gear, tuple(a.ctrlrange)) for a in acts], o, hfield=hfield,
                            plane=has_plane or hfield is None)
    return RigidModel(bodies, acts, o)
