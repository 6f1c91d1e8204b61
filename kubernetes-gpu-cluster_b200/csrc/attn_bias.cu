// Paged attention with a linear distance bias per head and a chunk mask, for any key / value head size, in bfloat16 or
// float32 storage.  One warp per (query row, head): 32 keys at a time, one key per lane for the scores (q in shared
// memory), softmax statistics in fp32 across the warp, then the lanes split the value columns.  Only keys of the
// query's own chunk are read, so the cost per query is bounded by the chunk size whatever the context length.
#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

constexpr int ATT_WARPS = 4, ATT_MAXV = 8;   // value columns per lane: vdim <= 32 * ATT_MAXV

template <typename E>
__global__ void __launch_bounds__(ATT_WARPS * 32) attn_bias_chunk_kernel(AttnBiasArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float qs_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * ATT_WARPS + warp;
  if (item >= (int64_t)a.T * a.H) return;
  const int t = (int)(item / a.H), h = (int)(item % a.H);
  float* qs = qs_all + warp * a.dim;
  const E* q = (const E*)a.q + (int64_t)t * a.ldq + h * a.dim;
  for (int d = lane; d < a.dim; d += 32) qs[d] = ldf(q + d);
  __syncwarp();
  const int b = a.token_req[t], i = a.positions[t];
  const int lo = a.chunk > 0 ? (i / a.chunk) * a.chunk : 0;
  const int g = h / (a.H / a.G);
  const float slope = a.bias_span > 0.f ? exp2f(-a.bias_span * (float)(h + 1) / (float)a.H) : 0.f;
  const int32_t* bt = a.block_table + (int64_t)b * a.max_blocks;
  const E* kc = (const E*)a.k_cache;
  const E* vc = (const E*)a.v_cache;
  float m = -INFINITY, l = 0.f, o[ATT_MAXV];
#pragma unroll
  for (int c = 0; c < ATT_MAXV; ++c) o[c] = 0.f;
  for (int j0 = lo; j0 <= i; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j <= i;
    int64_t row = 0;
    float s = -INFINITY;
    if (valid) {
      row = ((int64_t)bt[j / a.block_size] * a.G + g) * a.block_size + j % a.block_size;
      const E* kr = kc + row * a.dim;
      float acc = 0.f;
      for (int d = 0; d < a.dim; ++d) acc = fmaf(qs[d], ldf(kr + d), acc);
      s = acc * a.scale - slope * (float)(i - j);
    }
    const float mn = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - mn) : 0.f;
    const float corr = expf(m - mn);            // m = -inf on the first tile: exp(-inf) = 0
    l = l * corr + warp_sum(p);
    m = mn;
#pragma unroll
    for (int c = 0; c < ATT_MAXV; ++c) o[c] *= corr;
    const int cnt = min(32, i - j0 + 1);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int64_t rj = __shfl_sync(0xffffffffu, row, jj);
      const E* vr = vc + rj * a.vdim;
#pragma unroll
      for (int c = 0; c < ATT_MAXV; ++c) {
        const int col = c * 32 + lane;
        if (col < a.vdim) o[c] = fmaf(pj, ldf(vr + col), o[c]);
      }
    }
  }
  const float inv = a.out_scale / l;
  E* out = (E*)a.out + (int64_t)t * a.ldo + h * a.vdim;
#pragma unroll
  for (int c = 0; c < ATT_MAXV; ++c) {
    const int col = c * 32 + lane;
    if (col < a.vdim) stf(out + col, o[c] * inv);
  }
}

int attn_bias_chunk(const AttnBiasArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.vdim <= 32 * ATT_MAXV, "attn_bias_chunk: value head size %d > %d", a.vdim, 32 * ATT_MAXV);
  KGE_REQUIRE(a.dim <= 1024 && a.H % a.G == 0, "attn_bias_chunk: bad head sizes");
  const int64_t items = (int64_t)a.T * a.H;
  const dim3 grid((unsigned)((items + ATT_WARPS - 1) / ATT_WARPS)), block(ATT_WARPS * 32);
  const size_t smem = (size_t)ATT_WARPS * a.dim * 4;
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(attn_bias_chunk_kernel<float>, grid, block, smem, st, a)
                                        : launch_pdl(attn_bias_chunk_kernel<__nv_bfloat16>, grid, block, smem, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

template <typename E>
__global__ void kv_write_any_kernel(const E* k, int ldk, const E* v, int ldv, const int64_t* slots, E* kc, E* vc, int G, int dim, int vdim, int bs) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  const int64_t blk = slot / bs, off = slot % bs;
  for (int c = threadIdx.x; c < G * dim; c += blockDim.x) {
    const int g = c / dim, d = c % dim;
    kc[((blk * G + g) * bs + off) * dim + d] = k[(int64_t)t * ldk + c];
  }
  for (int c = threadIdx.x; c < G * vdim; c += blockDim.x) {
    const int g = c / vdim, d = c % vdim;
    vc[((blk * G + g) * bs + off) * vdim + d] = v[(int64_t)t * ldv + c];
  }
}

int kv_write_any(const void* k, int ldk, const void* v, int ldv, const int64_t* slots, void* k_cache, void* v_cache, int T, int G,
                 int dim, int vdim, int block_size, int elt, cudaStream_t st) {
  if (T <= 0) return 0;
  cudaError_t ce = elt == KGE_ELT_F32
      ? launch_pdl(kv_write_any_kernel<float>, dim3(T), dim3(128), 0, st, (const float*)k, ldk, (const float*)v, ldv, slots, (float*)k_cache, (float*)v_cache, G, dim, vdim, block_size)
      : launch_pdl(kv_write_any_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, st, (const __nv_bfloat16*)k, ldk, (const __nv_bfloat16*)v, ldv, slots,
                   (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, G, dim, vdim, block_size);
  KGE_CUDA_OK(ce);
  return 0;
}

}  // namespace kge
