// Rotary positions for layer-list models: partial (the first rot_dims dimensions of a head), interleaved pairs, plain
// or YaRN-scaled frequencies; fused with what surrounds the rotation in an attention mixer - an RMS norm over the whole
// q and k projections, the write of the rotated keys into the paged cache, and the write of the values (a projection of
// their own, or the un-normed, un-rotated key projection).  One block per token: sums of squares in fp32, the token's
// cos / sin pairs once in shared memory (angle = position * frequency formed in double precision, so long contexts
// lose nothing in the argument reduction), then every head reads them.
#include <math.h>

#include <algorithm>

#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

void rotary_frequencies(int dims, double base, double factor, double original, double fast, double slow, double* freq, float* mult) {
  const int half = dims / 2;
  for (int i = 0; i < half; ++i) freq[i] = pow(base, -2.0 * i / dims);
  *mult = 1.f;
  if (factor > 0.0) {
    const double pi = 3.14159265358979323846;
    auto corr = [&](double turns) { return dims * log(original / (2.0 * pi * turns)) / (2.0 * log(base)); };
    const double lo = std::max(floor(corr(fast)), 0.0), hi = std::min(ceil(corr(slow)), (double)(dims - 1));
    for (int i = 0; i < half; ++i) {
      const double ramp = std::min(std::max((i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
      freq[i] = freq[i] / factor * ramp + freq[i] * (1.0 - ramp);
    }
    *mult = (float)(0.1 * log(factor) + 1.0);
  }
}

template <typename E>
__global__ void __launch_bounds__(256) rotary_norm_kvwrite_kernel(RotaryArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float cs[];                 // [rot_dims / 2] cos, then sin (multiplier applied)
  __shared__ float red[33];
  const int t = blockIdx.x, half = a.rot_dims >> 1, nq = a.H * a.dim, nk = a.G * a.dim;
  const int pos = a.positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double s, c;
    sincos((double)pos * a.freq[i], &s, &c);
    cs[i] = (float)c * a.mult;
    cs[half + i] = (float)s * a.mult;
  }
  E* q = (E*)a.q + (int64_t)t * a.ldq;
  const E* k = (const E*)a.k + (int64_t)t * a.ldk;
  float inv_q = 1.f, inv_k = 1.f;
  if (a.q_norm_w) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < nq; c += blockDim.x) { const float v = ldf(q + c); ss = fmaf(v, v, ss); }
    inv_q = 1.f / sqrtf(block_sum(ss, red) / (float)nq + a.eps);
    __syncthreads();
  }
  if (a.k_norm_w) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < nk; c += blockDim.x) { const float v = ldf(k + c); ss = fmaf(v, v, ss); }
    inv_k = 1.f / sqrtf(block_sum(ss, red) / (float)nk + a.eps);
  }
  __syncthreads();
  const int64_t slot = a.slots ? a.slots[t] : -1;
  const int64_t blk = slot >= 0 ? slot / a.block_size : 0, off = slot >= 0 ? slot % a.block_size : 0;
  // values first: they may be the key projection as it came in
  if (slot >= 0 && a.v_cache) {
    const E* v = a.v ? (const E*)a.v + (int64_t)t * a.ldv : k;
    E* vc = (E*)a.v_cache;
    for (int c = threadIdx.x; c < a.G * a.vdim; c += blockDim.x) {
      const int g = c / a.vdim, d = c % a.vdim;
      vc[((blk * a.G + g) * a.block_size + off) * a.vdim + d] = v[c];
    }
  }
  // one item = one pair of neighbouring dimensions of one head (dim even), or the single last dimension of an odd head size
  const int ppd = (a.dim + 1) >> 1;
  for (int idx = threadIdx.x; idx < (a.H + a.G) * ppd; idx += blockDim.x) {
    const int hh = idx / ppd, pi = idx % ppd, d0 = 2 * pi;
    const bool isq = hh < a.H;
    const int head = isq ? hh : hh - a.H, col = head * a.dim + d0;
    const bool two = d0 + 1 < a.dim;
    const E* src = isq ? q : k;
    const E* nw = (const E*)(isq ? a.q_norm_w : a.k_norm_w);
    const float inv = isq ? inv_q : inv_k;
    float u = ldf(src + col) * inv, v = two ? ldf(src + col + 1) * inv : 0.f;
    if (nw) { u *= ldf(nw + col); if (two) v *= ldf(nw + col + 1); }
    if (d0 + 1 < a.rot_dims) {
      const float c = cs[pi], s = cs[half + pi];
      const float ru = u * c - v * s, rv = v * c + u * s;
      u = ru; v = rv;
    }
    if (isq) {
      stf(q + col, u); if (two) stf(q + col + 1, v);
    } else if (slot >= 0 && a.k_cache) {
      E* kc = (E*)a.k_cache + ((blk * a.G + head) * a.block_size + off) * a.dim + d0;
      stf(kc, u); if (two) stf(kc + 1, v);
    }
  }
}

int rotary_norm_kvwrite(const RotaryArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.q && a.k && a.positions && a.H > 0 && a.G > 0 && a.dim > 0 && a.rot_dims >= 0 && a.rot_dims <= a.dim && a.rot_dims % 2 == 0 &&
              (a.rot_dims == 0 || a.freq), "rotary_norm_kvwrite: bad arguments");
  KGE_REQUIRE(a.v || a.vdim == a.dim, "rotary_norm_kvwrite: values taken from the keys need vdim = dim");
  const size_t smem = (size_t)std::max(a.rot_dims, 2) * 4;
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(rotary_norm_kvwrite_kernel<float>, dim3(a.T), dim3(256), smem, st, a)
                                        : launch_pdl(rotary_norm_kvwrite_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), smem, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

}  // namespace kge
