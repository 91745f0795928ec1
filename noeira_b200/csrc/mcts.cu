// Batched MCTS tree operations, one thread per tree (root parallelisation): PUCT selection down to an unexpanded edge,
// and expansion of the evaluated leaf fused with the discounted backup along its path.  The tensor-program versions in
// planners/mcts.py (select_torch / expand_torch / backup_torch) are the oracle of the GPU test.
// Reference: noeira/planners/tree_search/mcts_gpu.mojo (selection / expand / backup kernels, 1 thread per env).
#include "common.cuh"

namespace {
using namespace nb;

__global__ void __launch_bounds__(128)
mcts_select_kernel(const int* __restrict__ children, const float* __restrict__ prior, const float* __restrict__ visit,
                   const float* __restrict__ value_sum, const float* __restrict__ reward, const float* __restrict__ minmax, int n,
                   int N, int A, float discount, float c_base, float c_init, int max_depth, int* leaf_parent, int* leaf_action) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const int* ch = children + (size_t)e * N * A;
  const float* pr = prior + (size_t)e * N * A;
  const float* vi = visit + (size_t)e * N;
  const float* vs = value_sum + (size_t)e * N;
  const float* rw = reward + (size_t)e * N;
  const float lo = minmax[e * 2], hi = minmax[e * 2 + 1];
  const bool span = hi > lo;
  const float inv = span ? 1.0f / fmaxf(hi - lo, 1e-8f) : 1.f;
  int node = 0, lp = 0, la = 0;
  bool done = false;
  for (int d = 0; d < max_depth && !done; ++d) {
    const float np = vi[node];
    const float c = logf((np + c_base + 1.f) / c_base) + c_init;
    const float sq = sqrtf(fmaxf(np, 1.f));
    float best = -INFINITY;
    int ba = 0;
    for (int a = 0; a < A; ++a) {
      const float p = pr[node * A + a];
      if (!(p > 0.f)) continue;
      const int c_ = ch[node * A + a];
      float nc = 0.f, q = 0.f;
      if (c_ >= 0) {
        nc = vi[c_];
        if (nc > 0.f) {
          const float qr = rw[c_] + discount * vs[c_] / fmaxf(nc, 1.f);
          q = span ? (qr - lo) * inv : qr;
        }
      }
      const float s = q + c * p * sq / (1.f + nc);
      if (s > best) { best = s; ba = a; }
    }
    const int child = ch[node * A + ba];
    if (child < 0) { lp = node; la = ba; done = true; }
    else node = child;
  }
  if (!done) { lp = node; la = 0; }
  leaf_parent[e] = lp;
  leaf_action[e] = la;
}

__global__ void __launch_bounds__(128)
mcts_expand_backup_kernel(int* children, float* prior, float* visit, float* value_sum, float* reward, int* parent, float* latent,
                          int* n_nodes, float* minmax, const int* __restrict__ leaf_parent, const int* __restrict__ leaf_action,
                          const float* __restrict__ new_latent, const float* __restrict__ new_reward,
                          const float* __restrict__ logits, const float* __restrict__ value, const unsigned char* __restrict__ legal,
                          int n, int N, int A, int L, float discount, int max_depth) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  int* ch = children + (size_t)e * N * A;
  float* pr = prior + (size_t)e * N * A;
  float* vi = visit + (size_t)e * N;
  float* vs = value_sum + (size_t)e * N;
  float* rw = reward + (size_t)e * N;
  int* pa = parent + (size_t)e * N;
  const int nn = min(n_nodes[e], N - 1);
  const int lp = leaf_parent[e], la = leaf_action[e];
  ch[lp * A + la] = nn;
  pa[nn] = lp;
  rw[nn] = new_reward[e];
  for (int i = 0; i < L; ++i) latent[((size_t)e * N + nn) * L + i] = new_latent[(size_t)e * L + i];
  // masked softmax of the leaf's policy logits
  float mx = -INFINITY;
  for (int a = 0; a < A; ++a)
    if (!legal || legal[(size_t)e * A + a]) mx = fmaxf(mx, logits[(size_t)e * A + a]);
  float sum = 0.f;
  for (int a = 0; a < A; ++a) {
    const float p = (!legal || legal[(size_t)e * A + a]) ? expf(logits[(size_t)e * A + a] - mx) : 0.f;
    pr[nn * A + a] = p;
    sum += p;
  }
  const float is = sum > 0.f ? 1.f / sum : 0.f;
  for (int a = 0; a < A; ++a) pr[nn * A + a] *= is;
  n_nodes[e] = nn + 1;
  // backup
  float g = value[e];
  float lo = minmax[e * 2], hi = minmax[e * 2 + 1];
  int node = nn;
  for (int d = 0; d < N; ++d) {   // a path has at most one node per simulation
    vs[node] += g;
    vi[node] += 1.f;
    if (node == 0) break;
    const float q = rw[node] + discount * (vs[node] / fmaxf(vi[node], 1.f));
    lo = fminf(lo, q);
    hi = fmaxf(hi, q);
    g = rw[node] + discount * g;
    node = pa[node];
  }
  minmax[e * 2] = lo;
  minmax[e * 2 + 1] = hi;
}

}  // namespace

extern "C" {

int nb_mcts_select(const int* children, const float* prior, const float* visit, const float* value_sum, const float* reward,
                   const float* minmax, int n, int N, int A, float discount, float c_base, float c_init, int max_depth,
                   int* leaf_parent, int* leaf_action, void* stream) {
  if (n <= 0 || A <= 0) return NB_ERR_BAD_ARG;
  mcts_select_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(children, prior, visit, value_sum, reward, minmax, n, N, A,
                                                                       discount, c_base, c_init, max_depth, leaf_parent, leaf_action);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_mcts_expand_backup(int* children, float* prior, float* visit, float* value_sum, float* reward, int* parent, float* latent,
                          int* n_nodes, float* minmax, const int* leaf_parent, const int* leaf_action, const float* new_latent,
                          const float* new_reward, const float* logits, const float* value, const unsigned char* legal, int n, int N,
                          int A, int L, float discount, int max_depth, void* stream) {
  if (n <= 0 || A <= 0) return NB_ERR_BAD_ARG;
  mcts_expand_backup_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      children, prior, visit, value_sum, reward, parent, latent, n_nodes, minmax, leaf_parent, leaf_action, new_latent, new_reward,
      logits, value, legal, n, N, A, L, discount, max_depth);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
