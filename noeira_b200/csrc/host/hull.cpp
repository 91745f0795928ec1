// 3-D convex hull by incremental insertion with horizon search (the role of noeira/physics3d/collision/native/nra_qhull.c,
// which calls libqhull_r; no qhull in this image, so the hull is computed here).  Output: outward-facing triangles.
#include <algorithm>
#include <cerrno>
#include <cmath>
#include <cstdint>
#include <map>
#include <vector>

#include "host_api.h"

namespace {
struct V3 { double x, y, z; };
inline V3 sub(V3 a, V3 b) { return {a.x - b.x, a.y - b.y, a.z - b.z}; }
inline V3 cross(V3 a, V3 b) { return {a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x}; }
inline double dot(V3 a, V3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
struct Face { int a, b, c; bool alive; };
}  // namespace

extern "C" int nbh_convex_hull(const double* xyz, int n, int32_t* tri_out, int max_tris) {
  if (n < 4) return -EINVAL;
  std::vector<V3> p(n);
  double scale = 0;
  for (int i = 0; i < n; ++i) {
    p[i] = {xyz[3 * i], xyz[3 * i + 1], xyz[3 * i + 2]};
    scale = std::max({scale, std::fabs(p[i].x), std::fabs(p[i].y), std::fabs(p[i].z)});
  }
  const double eps = 1e-10 * std::max(scale, 1.0);
  // initial tetrahedron: extreme pair, farthest from the line, farthest from the plane
  int i0 = 0, i1 = -1, i2 = -1, i3 = -1;
  for (int i = 1; i < n; ++i) if (p[i].x < p[i0].x) i0 = i;
  double best = 0;
  for (int i = 0; i < n; ++i) { const V3 d = sub(p[i], p[i0]); const double v = dot(d, d); if (v > best) { best = v; i1 = i; } }
  if (i1 < 0 || best < eps * eps) return -EINVAL;
  best = 0;
  for (int i = 0; i < n; ++i) { const V3 c = cross(sub(p[i1], p[i0]), sub(p[i], p[i0])); const double v = dot(c, c); if (v > best) { best = v; i2 = i; } }
  if (i2 < 0 || best < eps * eps) return -EINVAL;
  const V3 nrm = cross(sub(p[i1], p[i0]), sub(p[i2], p[i0]));
  best = 0;
  for (int i = 0; i < n; ++i) { const double v = std::fabs(dot(nrm, sub(p[i], p[i0]))); if (v > best) { best = v; i3 = i; } }
  if (i3 < 0 || best < eps * std::sqrt(dot(nrm, nrm))) return -EINVAL;
  std::vector<Face> faces;
  auto add_face = [&](int a, int b, int c, V3 inside) {
    // orient so that `inside` is behind the face
    const V3 nn = cross(sub(p[b], p[a]), sub(p[c], p[a]));
    if (dot(nn, sub(inside, p[a])) > 0) std::swap(b, c);
    faces.push_back({a, b, c, true});
  };
  const V3 centroid = {(p[i0].x + p[i1].x + p[i2].x + p[i3].x) / 4, (p[i0].y + p[i1].y + p[i2].y + p[i3].y) / 4,
                       (p[i0].z + p[i1].z + p[i2].z + p[i3].z) / 4};
  add_face(i0, i1, i2, centroid);
  add_face(i0, i1, i3, centroid);
  add_face(i0, i2, i3, centroid);
  add_face(i1, i2, i3, centroid);
  for (int i = 0; i < n; ++i) {
    if (i == i0 || i == i1 || i == i2 || i == i3) continue;
    std::vector<int> visible;
    for (int f = 0; f < (int)faces.size(); ++f) {
      if (!faces[f].alive) continue;
      const V3 nn = cross(sub(p[faces[f].b], p[faces[f].a]), sub(p[faces[f].c], p[faces[f].a]));
      if (dot(nn, sub(p[i], p[faces[f].a])) > eps * std::sqrt(dot(nn, nn))) visible.push_back(f);
    }
    if (visible.empty()) continue;          // inside or on the hull
    // horizon = directed edges of visible faces whose reverse edge is not in a visible face
    std::map<std::pair<int, int>, int> edges;
    for (int f : visible) {
      const int v[3] = {faces[f].a, faces[f].b, faces[f].c};
      for (int k = 0; k < 3; ++k) edges[{v[k], v[(k + 1) % 3]}] = 1;
    }
    for (int f : visible) faces[f].alive = false;
    for (const auto& e : edges) {
      if (edges.count({e.first.second, e.first.first})) continue;
      faces.push_back({e.first.first, e.first.second, i, true});   // keeps the visible face's winding
    }
  }
  int count = 0;
  for (const Face& f : faces) {
    if (!f.alive) continue;
    if (count >= max_tris) return -ERANGE;
    tri_out[3 * count] = f.a; tri_out[3 * count + 1] = f.b; tri_out[3 * count + 2] = f.c;
    ++count;
  }
  return count;
}
