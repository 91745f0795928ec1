// Convolution support kernels for the NHWC bf16 path: patch gather (im2col) feeding the tcgen05 GEMM,
// its adjoint as a deterministic gather (no atomics), BatchNorm2D in training mode (per-channel batch
// statistics, fused scale/shift/ReLU/residual), max pooling, and the uint8 camera-image normaliser.
//
// A convolution is  Y[B·OH·OW, OC] = col[B·OH·OW, KH·KW·C] · W[KH·KW·C, OC]  with the bias / ReLU in the GEMM
// epilogue; dgrad is  dcol = dY · Wᵀ  followed by the gather below; wgrad is  dW += colᵀ · dY  (TN GEMM).
// Reference: im2col + GEMM (noeira/nn/primitives/conv2d.mojo:437,652,723) or cuDNN (nn/core/cudnn_conv.mojo),
// BatchNorm 2-D NHWC kernels (batch_norm_2d.mojo:550-1250), max_pool_2d.mojo, act/data_gpu.mojo:157 (gather +
// /255 + ImageNet mean/std).
#include "common.cuh"

namespace {
using namespace nb;

// col[m, (kh*KW + kw)*C + c] = x[b, oh*s - p + kh, ow*s - p + kw, c]  (zero outside); C % 8 == 0, 16-byte copies
__global__ void __launch_bounds__(256)
im2col_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ col, int B, int H, int W, int C, int KH,
              int KW, int stride, int pad, int OH, int OW, int ldc) {
  const int cv = C / 8;
  const long long total = (long long)B * OH * OW * KH * KW * cv;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int c8 = (int)(i % cv);
    long long r = i / cv;
    const int kw = (int)(r % KW); r /= KW;
    const int kh = (int)(r % KH); r /= KH;
    const int ow = (int)(r % OW); r /= OW;
    const int oh = (int)(r % OH);
    const int b = (int)(r / OH);
    const int ih = oh * stride - pad + kh, iw = ow * stride - pad + kw;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (ih >= 0 && ih < H && iw >= 0 && iw < W)
      v = *reinterpret_cast<const uint4*>(x + (((size_t)b * H + ih) * W + iw) * C + c8 * 8);
    const size_t m = ((size_t)b * OH + oh) * OW + ow;
    *reinterpret_cast<uint4*>(col + m * ldc + ((size_t)kh * KW + kw) * C + c8 * 8) = v;
  }
}

// dx[b, h, w, c] = Σ_{kh,kw : (h+p-kh) % s == 0, ...} dcol[b, oh, ow, kh, kw, c]   (gather: one writer per element)
__global__ void __launch_bounds__(256)
col2im_kernel(const __nv_bfloat16* __restrict__ dcol, __nv_bfloat16* __restrict__ dx, int B, int H, int W, int C, int KH,
              int KW, int stride, int pad, int OH, int OW, int ldc) {
  const int cv = C / 8;
  const long long total = (long long)B * H * W * cv;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int c8 = (int)(i % cv);
    long long r = i / cv;
    const int w = (int)(r % W); r /= W;
    const int h = (int)(r % H);
    const int b = (int)(r / H);
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    for (int kh = 0; kh < KH; ++kh) {
      const int th = h + pad - kh;
      if (th < 0 || th % stride) continue;
      const int oh = th / stride;
      if (oh >= OH) continue;
      for (int kw = 0; kw < KW; ++kw) {
        const int tw = w + pad - kw;
        if (tw < 0 || tw % stride) continue;
        const int ow = tw / stride;
        if (ow >= OW) continue;
        const size_t m = ((size_t)b * OH + oh) * OW + ow;
        const uint4 v = *reinterpret_cast<const uint4*>(dcol + m * ldc + ((size_t)kh * KW + kw) * C + c8 * 8);
        const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          acc[2 * k] += __low2float(hp[k]);
          acc[2 * k + 1] += __high2float(hp[k]);
        }
      }
    }
    uint4 o;
    __nv_bfloat162 h0 = __floats2bfloat162_rn(acc[0], acc[1]), h1 = __floats2bfloat162_rn(acc[2], acc[3]),
                   h2 = __floats2bfloat162_rn(acc[4], acc[5]), h3 = __floats2bfloat162_rn(acc[6], acc[7]);
    o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
    o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(dx + (((size_t)b * H + h) * W + w) * C + c8 * 8) = o;
  }
}

// ---- BatchNorm2D over an [M, C] view (M = B·H·W).  Stage 1: per-slab Σx, Σx² (or Σdy, Σdy·x̂ for the backward).
__global__ void __launch_bounds__(256)
bn_reduce_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b2, const float* __restrict__ mean,
                 const float* __restrict__ rstd, float* __restrict__ p0, float* __restrict__ p1, int M, int C,
                 int rows_per_block, int mode /*0: Σa, Σa² ; 1: Σa, Σa·x̂(b2) */, const __nv_bfloat16* __restrict__ relu_out) {
  // L lanes (of 8 channels each) span a row; the other 256 / L thread groups take different rows, so that narrow
  // layers (C = 64: L = 8, 32 rows per sweep) keep every lane loading
  __shared__ float s0[256][9], s1[256][9];
  int L = 1;
  while (L < 32 && L * 8 < C) L <<= 1;
  const int R = 256 / L;
  const int cg = threadIdx.x % L, rg = threadIdx.x / L;
  const int col = blockIdx.x * 256 + cg * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(M, r0 + rows_per_block);
  float a0[8], a1[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) a0[k] = a1[k] = 0.f;
  if (col < C) {
    for (int r = r0 + rg; r < r1; r += R) {
      const uint4 va = __ldg(reinterpret_cast<const uint4*>(a + (size_t)r * C + col));
      const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&va);
      float fa[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) { fa[2 * k] = __low2float(ha[k]); fa[2 * k + 1] = __high2float(ha[k]); }
      if (mode == 0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) { a0[k] += fa[k]; a1[k] += fa[k] * fa[k]; }
      } else {
        const uint4 vb = __ldg(reinterpret_cast<const uint4*>(b2 + (size_t)r * C + col));
        const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&vb);
        uint4 vo = make_uint4(0, 0, 0, 0);
        if (relu_out) vo = __ldg(reinterpret_cast<const uint4*>(relu_out + (size_t)r * C + col));
        const __nv_bfloat162* ho = reinterpret_cast<const __nv_bfloat162*>(&vo);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float x0 = __low2float(hb[k]), x1 = __high2float(hb[k]);
          float d0 = fa[2 * k], d1 = fa[2 * k + 1];
          if (relu_out) {
            if (!(__low2float(ho[k]) > 0.f)) d0 = 0.f;
            if (!(__high2float(ho[k]) > 0.f)) d1 = 0.f;
          }
          a0[2 * k] += d0; a0[2 * k + 1] += d1;
          a1[2 * k] += d0 * (x0 - mean[col + 2 * k]) * rstd[col + 2 * k];
          a1[2 * k + 1] += d1 * (x1 - mean[col + 2 * k + 1]) * rstd[col + 2 * k + 1];
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) { s0[threadIdx.x][k] = a0[k]; s1[threadIdx.x][k] = a1[k]; }
  __syncthreads();
  if ((int)threadIdx.x < L * 8) {
    float t0 = 0.f, t1 = 0.f;
    const int lane_of_col = threadIdx.x >> 3, k = threadIdx.x & 7;
    for (int g = 0; g < R; ++g) { t0 += s0[g * L + lane_of_col][k]; t1 += s1[g * L + lane_of_col][k]; }
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < C) { p0[(size_t)blockIdx.y * C + c] = t0; p1[(size_t)blockIdx.y * C + c] = t1; }
  }
}

// forward finish: mean, rstd, running stats
__global__ void bn_stats_finish_kernel(const float* __restrict__ p0, const float* __restrict__ p1, int split, int M, int C,
                                       float eps, float momentum, float* __restrict__ mean, float* __restrict__ rstd,
                                       float* __restrict__ run_mean, float* __restrict__ run_var) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f, ss = 0.f;
  for (int k = 0; k < split; ++k) { s += p0[(size_t)k * C + c]; ss += p1[(size_t)k * C + c]; }
  const float mu = s / M, var = fmaxf(ss / M - mu * mu, 0.f);
  mean[c] = mu;
  rstd[c] = rsqrtf(var + eps);
  if (run_mean) {
    run_mean[c] = (1.f - momentum) * run_mean[c] + momentum * mu;
    run_var[c] = (1.f - momentum) * run_var[c] + momentum * var * ((float)M / fmaxf(M - 1.f, 1.f));
  }
}
// backward finish: dgamma += Σdy·x̂, dbeta += Σdy ; keeps the sums for the dx kernel
__global__ void bn_bwd_finish_kernel(const float* __restrict__ p0, const float* __restrict__ p1, int split, int C,
                                     float* __restrict__ sum_dy, float* __restrict__ sum_dyx, float* __restrict__ dgamma,
                                     float* __restrict__ dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f, ss = 0.f;
  for (int k = 0; k < split; ++k) { s += p0[(size_t)k * C + c]; ss += p1[(size_t)k * C + c]; }
  sum_dy[c] = s;
  sum_dyx[c] = ss;
  if (dgamma) dgamma[c] += ss;
  if (dbeta) dbeta[c] += s;
}

// y = relu?( (x - mean) * rstd * gamma + beta + residual? )
__global__ void __launch_bounds__(256)
bn_apply_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ mean, const float* __restrict__ rstd,
                const float* __restrict__ gamma, const float* __restrict__ beta, const __nv_bfloat16* __restrict__ res,
                __nv_bfloat16* __restrict__ y, long long M, int C, int relu) {
  const int cv = C / 8;
  const long long total = M * cv, step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int c0 = (int)(i % cv) * 8;
    const uint4 vx = *reinterpret_cast<const uint4*>(x + i * 8);
    const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&vx);
    uint4 vr = make_uint4(0, 0, 0, 0);
    if (res) vr = *reinterpret_cast<const uint4*>(res + i * 8);
    const __nv_bfloat162* hr = reinterpret_cast<const __nv_bfloat162*>(&vr);
    float o[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + 2 * k;
      o[2 * k] = (__low2float(hx[k]) - mean[c]) * rstd[c] * gamma[c] + beta[c] + __low2float(hr[k]);
      o[2 * k + 1] = (__high2float(hx[k]) - mean[c + 1]) * rstd[c + 1] * gamma[c + 1] + beta[c + 1] + __high2float(hr[k]);
      if (relu) { o[2 * k] = fmaxf(o[2 * k], 0.f); o[2 * k + 1] = fmaxf(o[2 * k + 1], 0.f); }
    }
    uint4 vo;
    __nv_bfloat162 h0 = __floats2bfloat162_rn(o[0], o[1]), h1 = __floats2bfloat162_rn(o[2], o[3]),
                   h2 = __floats2bfloat162_rn(o[4], o[5]), h3 = __floats2bfloat162_rn(o[6], o[7]);
    vo.x = *reinterpret_cast<uint32_t*>(&h0); vo.y = *reinterpret_cast<uint32_t*>(&h1);
    vo.z = *reinterpret_cast<uint32_t*>(&h2); vo.w = *reinterpret_cast<uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(y + i * 8) = vo;
  }
}

// dx = gamma·rstd·( g − Σg/M − x̂·Σ(g·x̂)/M ),  g = dy masked by the ReLU output; dres = g (residual branch)
__global__ void __launch_bounds__(256)
bn_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                 const __nv_bfloat16* __restrict__ relu_out, const float* __restrict__ mean,
                 const float* __restrict__ rstd, const float* __restrict__ gamma, const float* __restrict__ sum_dy,
                 const float* __restrict__ sum_dyx, __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dres,
                 long long M, int C) {
  const int cv = C / 8;
  const float invM = 1.f / (float)M;
  const long long total = M * cv, step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int c0 = (int)(i % cv) * 8;
    const uint4 vd = *reinterpret_cast<const uint4*>(dy + i * 8), vx = *reinterpret_cast<const uint4*>(x + i * 8);
    uint4 vo = make_uint4(0, 0, 0, 0);
    if (relu_out) vo = *reinterpret_cast<const uint4*>(relu_out + i * 8);
    const __nv_bfloat16* hd = reinterpret_cast<const __nv_bfloat16*>(&vd);
    const __nv_bfloat16* hx = reinterpret_cast<const __nv_bfloat16*>(&vx);
    const __nv_bfloat16* ho = reinterpret_cast<const __nv_bfloat16*>(&vo);
    __nv_bfloat16 od[8], og[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int c = c0 + k;
      float g = __bfloat162float(hd[k]);
      if (relu_out && !(__bfloat162float(ho[k]) > 0.f)) g = 0.f;
      const float xh = (__bfloat162float(hx[k]) - mean[c]) * rstd[c];
      od[k] = __float2bfloat16(gamma[c] * rstd[c] * (g - sum_dy[c] * invM - xh * sum_dyx[c] * invM));
      og[k] = __float2bfloat16(g);
    }
    *reinterpret_cast<uint4*>(dx + i * 8) = *reinterpret_cast<uint4*>(od);
    if (dres) *reinterpret_cast<uint4*>(dres + i * 8) = *reinterpret_cast<uint4*>(og);
  }
}

// Average pooling with window K, stride = K (non-overlapping) on NHWC: forward averages, backward spreads dy / K².
// `back != 0`: `src` is dy [B, OH, OW, C] and `dst` is dx [B, H, W, C] (pixels outside the pooled area get zero).
__global__ void __launch_bounds__(256)
avgpool_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int B, int H, int W, int C, int K, int OH,
               int OW, int back) {
  const long long total = back ? (long long)B * H * W * C : (long long)B * OH * OW * C, step = (long long)gridDim.x * blockDim.x;
  const float inv = 1.f / (float)(K * K);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int c = (int)(i % C);
    long long r = i / C;
    if (back) {
      const int w = (int)(r % W); r /= W;
      const int h = (int)(r % H);
      const int b = (int)(r / H);
      const int oh = h / K, ow = w / K;
      dst[i] = (oh < OH && ow < OW) ? __float2bfloat16(__bfloat162float(src[(((long long)b * OH + oh) * OW + ow) * C + c]) * inv)
                                    : __float2bfloat16(0.f);
    } else {
      const int ow = (int)(r % OW); r /= OW;
      const int oh = (int)(r % OH);
      const int b = (int)(r / OH);
      float acc = 0.f;
      for (int kh = 0; kh < K; ++kh)
        for (int kw = 0; kw < K; ++kw)
          acc += __bfloat162float(src[(((long long)b * H + oh * K + kh) * W + ow * K + kw) * C + c]);
      dst[i] = __float2bfloat16(acc * inv);
    }
  }
}
// Nearest-neighbour upsampling by an integer factor S on NHWC: forward replicates, backward sums the S x S block.
__global__ void __launch_bounds__(256)
upsample_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, int B, int H, int W, int C, int S, int back) {
  const int OH = H * S, OW = W * S;
  const long long total = back ? (long long)B * H * W * C : (long long)B * OH * OW * C, step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int c = (int)(i % C);
    long long r = i / C;
    if (back) {
      const int w = (int)(r % W); r /= W;
      const int h = (int)(r % H);
      const int b = (int)(r / H);
      float acc = 0.f;
      for (int kh = 0; kh < S; ++kh)
        for (int kw = 0; kw < S; ++kw)
          acc += __bfloat162float(src[(((long long)b * OH + h * S + kh) * OW + w * S + kw) * C + c]);
      dst[i] = __float2bfloat16(acc);
    } else {
      const int ow = (int)(r % OW); r /= OW;
      const int oh = (int)(r % OH);
      const int b = (int)(r / OH);
      dst[i] = src[(((long long)b * H + oh / S) * W + ow / S) * C + c];
    }
  }
}

// 3x3 / stride 2 / pad 1 style max pooling on NHWC; idx stores the flat input offset of the maximum
__global__ void __launch_bounds__(256)
maxpool_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, int* __restrict__ idx, int B, int H,
                   int W, int C, int K, int stride, int pad, int OH, int OW) {
  const long long total = (long long)B * OH * OW * C, step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int c = (int)(i % C);
    long long r = i / C;
    const int ow = (int)(r % OW); r /= OW;
    const int oh = (int)(r % OH);
    const int b = (int)(r / OH);
    float best = -INFINITY;
    int bi = -1;
    for (int kh = 0; kh < K; ++kh) {
      const int ih = oh * stride - pad + kh;
      if (ih < 0 || ih >= H) continue;
      for (int kw = 0; kw < K; ++kw) {
        const int iw = ow * stride - pad + kw;
        if (iw < 0 || iw >= W) continue;
        const int off = ((b * H + ih) * W + iw) * C + c;
        const float v = __bfloat162float(x[off]);
        if (v > best) { best = v; bi = off; }
      }
    }
    y[i] = __float2bfloat16(best);
    idx[i] = bi;
  }
}
// dx = gather over the windows that contain the element (at most ceil(K/stride)^2 = 4 for 3x3 / 2): deterministic.
// One thread owns 8 consecutive channels of one input pixel when C % 8 == 0 (16-byte dy loads, 32-byte idx loads);
// the candidate output range is computed directly instead of testing all K*K taps.
template <int VEC>
__global__ void __launch_bounds__(256)
maxpool_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const int* __restrict__ idx, __nv_bfloat16* __restrict__ dx, int B,
                   int H, int W, int C, int K, int stride, int pad, int OH, int OW) {
  const int CV = C / VEC;
  const long long total = (long long)B * H * W * CV, step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const int cv = (int)(i % CV);
    long long r = i / CV;
    const int w = (int)(r % W); r /= W;
    const int h = (int)(r % H);
    const int b = (int)(r / H);
    const int c0 = cv * VEC;
    const int my = ((b * H + h) * W + w) * C + c0;
    // output rows oh with oh*stride - pad <= h <= oh*stride - pad + K - 1
    const int oh_lo = max(0, (h + pad - K + stride) / stride), oh_hi = min(OH - 1, (h + pad) / stride);
    const int ow_lo = max(0, (w + pad - K + stride) / stride), ow_hi = min(OW - 1, (w + pad) / stride);
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    for (int oh = oh_lo; oh <= oh_hi; ++oh)
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        const long long o = (((long long)b * OH + oh) * OW + ow) * C + c0;
        if (VEC == 8) {
          const int4 i0 = *reinterpret_cast<const int4*>(idx + o), i1 = *reinterpret_cast<const int4*>(idx + o + 4);
          const uint4 g = *reinterpret_cast<const uint4*>(dy + o);
          const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
          const int id[8] = {i0.x, i0.y, i0.z, i0.w, i1.x, i1.y, i1.z, i1.w};
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float gv = (j & 1) ? __high2float(gh[j >> 1]) : __low2float(gh[j >> 1]);
            if (id[j] == my + j) acc[j] += gv;
          }
        } else {
          if (idx[o] == my) acc[0] += __bfloat162float(dy[o]);
        }
      }
    if (VEC == 8) {
      uint4 out;
      __nv_bfloat162* oh2 = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      *reinterpret_cast<uint4*>(dx + my) = out;
    } else {
      dx[my] = __float2bfloat16(acc[0]);
    }
  }
}

// uint8 [B, 3, H, W] (CHW camera frames) → bf16 NHWC with C padded to 8: (x/255 − mean) / std
__global__ void __launch_bounds__(256)
image_normalize_kernel(const unsigned char* __restrict__ img, __nv_bfloat16* __restrict__ out, int B, int H, int W,
                       float m0, float m1, float m2, float s0, float s1, float s2) {
  const long long total = (long long)B * H * W, step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const long long hw = i % ((long long)H * W), b = i / ((long long)H * W);
    const unsigned char* p = img + b * 3 * H * W + hw;
    __nv_bfloat16 o[8];
    o[0] = __float2bfloat16((p[0] * (1.f / 255.f) - m0) / s0);
    o[1] = __float2bfloat16((p[(long long)H * W] * (1.f / 255.f) - m1) / s1);
    o[2] = __float2bfloat16((p[2LL * H * W] * (1.f / 255.f) - m2) / s2);
#pragma unroll
    for (int k = 3; k < 8; ++k) o[k] = __float2bfloat16(0.f);
    *reinterpret_cast<uint4*>(out + i * 8) = *reinterpret_cast<uint4*>(o);
  }
}

inline int g1(long long n) {
  long long b = (n + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}
}  // namespace

extern "C" {

int nb_im2col(const void* x, void* col, int B, int H, int W, int C, int KH, int KW, int stride, int pad, int OH, int OW,
              int ldc, void* stream) {
  if (C % 8 || ldc % 8) return NB_ERR_UNALIGNED;
  im2col_kernel<<<g1((long long)B * OH * OW * KH * KW * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)col, B, H, W, C, KH, KW, stride, pad, OH, OW, ldc);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
int nb_col2im(const void* dcol, void* dx, int B, int H, int W, int C, int KH, int KW, int stride, int pad, int OH, int OW,
              int ldc, void* stream) {
  if (C % 8 || ldc % 8) return NB_ERR_UNALIGNED;
  col2im_kernel<<<g1((long long)B * H * W * (C / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dcol, (__nv_bfloat16*)dx, B, H, W, C, KH, KW, stride, pad, OH, OW, ldc);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_bn_split(long long M) {
  long long s = M / 256;
  return (int)(s < 1 ? 1 : (s > 1024 ? 1024 : s));
}
// partials: 2 * nb_bn_split(M) * C floats
int nb_bn_fwd(const void* x, const float* gamma, const float* beta, const void* residual, void* y, float* mean, float* rstd,
              float* run_mean, float* run_var, float* partials, long long M, int C, float eps, float momentum, int relu,
              int training, void* stream) {
  if (C % 8) return NB_ERR_UNALIGNED;
  cudaStream_t s = (cudaStream_t)stream;
  if (training) {
    const int split = nb_bn_split(M);
    const int rows = (int)ceil_div_ll(M, split);
    float* p0 = partials;
    float* p1 = partials + (size_t)split * C;
    bn_reduce_kernel<<<dim3(ceil_div(C, 256), (unsigned)ceil_div_ll(M, rows)), 256, 0, s>>>(
        (const __nv_bfloat16*)x, nullptr, nullptr, nullptr, p0, p1, (int)M, C, rows, 0, nullptr);
    NB_LAUNCH_CHECK();
    bn_stats_finish_kernel<<<ceil_div(C, 128), 128, 0, s>>>(p0, p1, (int)ceil_div_ll(M, rows), (int)M, C, eps, momentum,
                                                           mean, rstd, run_mean, run_var);
    NB_LAUNCH_CHECK();
  }
  bn_apply_kernel<<<g1(M * (C / 8)), 256, 0, s>>>((const __nv_bfloat16*)x, mean, rstd, gamma, beta,
                                                 (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, M, C, relu);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
// relu_out: the forward output when ReLU was fused (masks dy), else null.  sums: 2*C floats of scratch.
int nb_bn_bwd(const void* dy, const void* x, const void* relu_out, const float* mean, const float* rstd,
              const float* gamma, void* dx, void* dres, float* dgamma, float* dbeta, float* partials, float* sums,
              long long M, int C, void* stream) {
  if (C % 8) return NB_ERR_UNALIGNED;
  cudaStream_t s = (cudaStream_t)stream;
  const int split = nb_bn_split(M);
  const int rows = (int)ceil_div_ll(M, split);
  float* p0 = partials;
  float* p1 = partials + (size_t)split * C;
  bn_reduce_kernel<<<dim3(ceil_div(C, 256), (unsigned)ceil_div_ll(M, rows)), 256, 0, s>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, mean, rstd, p0, p1, (int)M, C, rows, 1,
      (const __nv_bfloat16*)relu_out);
  NB_LAUNCH_CHECK();
  bn_bwd_finish_kernel<<<ceil_div(C, 128), 128, 0, s>>>(p0, p1, (int)ceil_div_ll(M, rows), C, sums, sums + C, dgamma, dbeta);
  NB_LAUNCH_CHECK();
  bn_bwd_dx_kernel<<<g1(M * (C / 8)), 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                  (const __nv_bfloat16*)relu_out, mean, rstd, gamma, sums, sums + C,
                                                  (__nv_bfloat16*)dx, (__nv_bfloat16*)dres, M, C);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_maxpool_fwd(const void* x, void* y, int* idx, int B, int H, int W, int C, int K, int stride, int pad, int OH, int OW,
                   void* stream) {
  maxpool_fwd_kernel<<<g1((long long)B * OH * OW * C), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, idx, B, H, W, C, K, stride, pad, OH, OW);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
int nb_maxpool_bwd(const void* dy, const int* idx, void* dx, int B, int H, int W, int C, int K, int stride, int pad, int OH,
                   int OW, void* stream) {
  if (C % 8 == 0)
    maxpool_bwd_kernel<8><<<g1((long long)B * H * W * C / 8), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)dy, idx, (__nv_bfloat16*)dx, B, H, W, C, K, stride, pad, OH, OW);
  else
    maxpool_bwd_kernel<1><<<g1((long long)B * H * W * C), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, idx, (__nv_bfloat16*)dx, B, H, W, C, K, stride, pad, OH, OW);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
int nb_avgpool(const void* src, void* dst, int B, int H, int W, int C, int K, int OH, int OW, int back, void* stream) {
  if (K <= 0 || OH * K > H || OW * K > W) return NB_ERR_BAD_ARG;
  const long long total = back ? (long long)B * H * W * C : (long long)B * OH * OW * C;
  avgpool_kernel<<<g1(total), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, B, H, W, C, K, OH, OW, back);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
// H, W are the LOW-resolution sizes in both directions
int nb_upsample_nearest(const void* src, void* dst, int B, int H, int W, int C, int S, int back, void* stream) {
  if (S <= 0) return NB_ERR_BAD_ARG;
  const long long total = back ? (long long)B * H * W * C : (long long)B * H * S * W * S * C;
  upsample_kernel<<<g1(total), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, B, H, W, C, S, back);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
int nb_image_normalize(const unsigned char* img, void* out, int B, int H, int W, float m0, float m1, float m2, float s0,
                       float s1, float s2, void* stream) {
  image_normalize_kernel<<<g1((long long)B * H * W), 256, 0, (cudaStream_t)stream>>>(img, (__nv_bfloat16*)out, B, H, W, m0,
                                                                                  m1, m2, s0, s1, s2);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
