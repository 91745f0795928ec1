// Per-epoch crop + flip augmentation of a resident image set: out[n] = flip?(crop(pad(raw[n]), dx, dy)), one draw per
// (sample, epoch) from a counter hash (training/augment.py::crop_flip_draws is the same arithmetic).  One thread per
// output element, NCHW or NHWC, fp32 or bf16.  Reference: noeira/nn/training/augmenter.mojo:70-200.
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned int hash_u32(unsigned int x) {
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
  return x;
}

template <typename T>
__global__ void __launch_bounds__(256)
crop_flip_kernel(const T* __restrict__ raw, T* __restrict__ out, int N, int C, int H, int W, int pad, int nhwc, unsigned int epoch,
                 unsigned int seed) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)N * C * H * W;
  if (idx >= total) return;
  int n, c, y, x;
  if (nhwc) {
    c = (int)(idx % C); x = (int)((idx / C) % W); y = (int)((idx / ((long long)C * W)) % H); n = (int)(idx / ((long long)C * W * H));
  } else {
    x = (int)(idx % W); y = (int)((idx / W) % H); c = (int)((idx / ((long long)W * H)) % C); n = (int)(idx / ((long long)W * H * C));
  }
  const unsigned int h = hash_u32((unsigned int)n * 0x9E3779B1u + epoch * 0x85EBCA77u + seed * 0xC2B2AE3Du);
  const unsigned int span = 2u * (unsigned int)pad + 1u;
  const int dx = (int)(h % span), dy = (int)((h >> 8) % span), flip = (int)((h >> 20) & 1u);
  const int sx = (flip ? W - 1 - x : x) + dx - pad, sy = y + dy - pad;
  T v = T(0.f);
  if (sx >= 0 && sx < W && sy >= 0 && sy < H) {
    const long long s = nhwc ? (((long long)n * H + sy) * W + sx) * C + c : (((long long)n * C + c) * H + sy) * W + sx;
    v = raw[s];
  }
  out[idx] = v;
}

}  // namespace

extern "C" int nb_augment_crop_flip(const void* raw, void* out, int N, int C, int H, int W, int pad, int nhwc, int bf16,
                                    unsigned int epoch, unsigned int seed, void* stream) {
  if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || pad < 0) return NB_ERR_BAD_ARG;
  const long long total = (long long)N * C * H * W;
  const unsigned int grid = (unsigned int)((total + 255) / 256);
  if (bf16)
    crop_flip_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)raw, (__nv_bfloat16*)out, N, C, H, W,
                                                                           pad, nhwc, epoch, seed);
  else
    crop_flip_kernel<float><<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)raw, (float*)out, N, C, H, W, pad, nhwc, epoch, seed);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
