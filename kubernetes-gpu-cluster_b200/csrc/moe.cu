// Mixture-of-experts routing: fp32 router logits (optional bias), sigmoid or softmax scores or the raw logits with a
// softmax over the chosen ones, top-k choice, and the grouping of
// (token, choice) pairs by expert that the grouped linear layer consumes.  Which rows an expert gets is all that the
// grouping decides: a pair's result does not depend on its place in the group, and the pairs of a token are summed in
// choice order afterwards, so the routing order never shows in the output.
#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

// One block per token: its eight warps share the experts' dot products (fp32, ascending d per lane, lanes summed by
// shuffles - the same order whatever the launch holds), then one thread picks the top-k.
template <typename E>
__global__ void __launch_bounds__(256) moe_score_kernel(MoeRouteArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sc[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = blockIdx.x;
  const E* h = (const E*)a.h + (int64_t)t * a.ldh;
  for (int e = warp; e < a.E; e += 8) {
    const E* w = (const E*)a.w_router + (int64_t)e * a.d;
    float acc = 0.f;
#pragma unroll 8
    for (int k = lane; k < a.d; k += 32) acc = fmaf(ldf(h + k), ldf(w + k), acc);
    acc = warp_sum(acc);
    if (lane == 0) sc[e] = a.b_router ? acc + ldf((const E*)a.b_router + e) : acc;
  }
  __syncthreads();
  if (warp != 0) return;
  if (a.score_fn == 0) {
    for (int e = lane; e < a.E; e += 32) sc[e] = 1.f / (1.f + expf(-sc[e]));
  } else if (a.score_fn == 1) {
    float mx = -INFINITY;
    for (int e = lane; e < a.E; e += 32) mx = fmaxf(mx, sc[e]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < a.E; e += 32) { const float p = expf(sc[e] - mx); sc[e] = p; sum += p; }
    sum = warp_sum(sum);
    __syncwarp();
    for (int e = lane; e < a.E; e += 32) sc[e] /= sum;
  }
  __syncwarp();
  if (lane == 0) {
    float total = 0.f;
    for (int k = 0; k < a.top; ++k) {
      int best = -1; float bv = -INFINITY;
      for (int e = 0; e < a.E; ++e) {
        bool taken = false;
        for (int q = 0; q < k; ++q) taken |= a.choice_expert[(int64_t)t * a.top + q] == e;
        if (!taken && sc[e] > bv) { bv = sc[e]; best = e; }
      }
      if (best < 0) { best = 0; for (int q = 0; q < k; ++q) if (a.choice_expert[(int64_t)t * a.top + q] == best) ++best; bv = 0.f; }   // scores that are not numbers
      a.choice_expert[(int64_t)t * a.top + k] = best;
      a.choice_weight[(int64_t)t * a.top + k] = bv;
      total += bv;
    }
    if (a.score_fn == 2) {          // softmax over the chosen logits only (the first choice holds the largest)
      const float mx = a.choice_weight[(int64_t)t * a.top];
      total = 0.f;
      for (int k = 0; k < a.top; ++k) { const float p = expf(a.choice_weight[(int64_t)t * a.top + k] - mx); a.choice_weight[(int64_t)t * a.top + k] = p; total += p; }
      for (int k = 0; k < a.top; ++k) a.choice_weight[(int64_t)t * a.top + k] /= total;
    } else if (a.renorm) for (int k = 0; k < a.top; ++k) a.choice_weight[(int64_t)t * a.top + k] /= total;
  }
}

__global__ void __launch_bounds__(1024) moe_group_kernel(MoeRouteArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int cnt[];            // [E] counts, then [E] cursors
  int* cur = cnt + a.E;
  const int n = a.T * a.top;
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[a.choice_expert[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < a.E; ++e) {
      a.group_off[e] = off; cur[e] = off;
      off += a.pad > 1 ? (cnt[e] + a.pad - 1) / a.pad * a.pad : cnt[e];
    }
    a.group_off[a.E] = off;
  }
  __syncthreads();
  if (a.pad > 1) {
    // padded groups: rows that carry no pair are marked (the gather writes zeros there, the scatter skips them), and every
    // tile of `pad` rows learns its expert; tiles beyond the last group compute on zero rows with the first expert's weights
    for (int i = threadIdx.x; i < a.rows_padded; i += blockDim.x) { a.perm_token[i] = -1; a.perm_dest[i] = -1; a.perm_weight[i] = 0.f; }
    for (int i = threadIdx.x; i < a.rows_padded / a.pad; i += blockDim.x) {
      int e = 0;
      while (e + 1 < a.E && i * a.pad >= a.group_off[e + 1]) ++e;
      a.tile_group[i] = i * a.pad < a.group_off[a.E] ? e : 0;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int p = atomicAdd(&cur[a.choice_expert[i]], 1);
    a.perm_token[p] = i / a.top;
    a.perm_weight[p] = a.choice_weight[i];
    a.perm_dest[p] = i;
  }
}

__global__ void moe_gather_rows_kernel(__nv_bfloat16* xperm, const __nv_bfloat16* h, int ldh, const int32_t* tok, const float* w, int d) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x;
  if (tok[p] < 0) {                              // a padding row of a group
    for (int c = threadIdx.x; c < d; c += blockDim.x) xperm[(int64_t)p * d + c] = __float2bfloat16_rn(0.f);
    return;
  }
  const __nv_bfloat16* src = h + (int64_t)tok[p] * ldh;
  if (!w && d % 8 == 0 && ldh % 8 == 0) {        // plain copy of the row, 16 bytes at a time
    for (int c = threadIdx.x; c < d / 8; c += blockDim.x) reinterpret_cast<uint4*>(xperm + (int64_t)p * d)[c] = reinterpret_cast<const uint4*>(src)[c];
    return;
  }
  const float s = w ? w[p] : 1.f;
  for (int c = threadIdx.x; c < d; c += blockDim.x) xperm[(int64_t)p * d + c] = __float2bfloat16_rn(s * __bfloat162float(src[c]));
}
__global__ void moe_scatter_rows_kernel(__nv_bfloat16* out, const __nv_bfloat16* operm, const int32_t* dest, int d) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = blockIdx.x;
  if (dest[p] < 0) return;
  if (d % 8 == 0) {
    for (int c = threadIdx.x; c < d / 8; c += blockDim.x) reinterpret_cast<uint4*>(out + (int64_t)dest[p] * d)[c] = reinterpret_cast<const uint4*>(operm + (int64_t)p * d)[c];
    return;
  }
  for (int c = threadIdx.x; c < d; c += blockDim.x) out[(int64_t)dest[p] * d + c] = operm[(int64_t)p * d + c];
}
int moe_gather_rows(void* xperm, const void* h, int ldh, const int32_t* perm_token, const float* perm_weight, int np, int d, cudaStream_t st) {
  if (np <= 0) return 0;
  KGE_CUDA_OK(launch_pdl(moe_gather_rows_kernel, dim3(np), dim3(256), 0, st, (__nv_bfloat16*)xperm, (const __nv_bfloat16*)h, ldh, perm_token, perm_weight, d));
  return 0;
}
int moe_scatter_rows(void* out, const void* operm, const int32_t* perm_dest, int np, int d, cudaStream_t st) {
  if (np <= 0) return 0;
  KGE_CUDA_OK(launch_pdl(moe_scatter_rows_kernel, dim3(np), dim3(256), 0, st, (__nv_bfloat16*)out, (const __nv_bfloat16*)operm, perm_dest, d));
  return 0;
}

int moe_route(const MoeRouteArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.E > 0 && a.top > 0 && a.top <= a.E && a.E <= 4096, "moe_route: %d experts, top %d", a.E, a.top);
  KGE_REQUIRE(a.pad <= 1 || (a.tile_group && a.rows_padded % a.pad == 0 && a.rows_padded >= a.T * a.top + a.E * (a.pad - 1)),
              "moe_route: padded groups need tile_group and %d rows or more", a.T * a.top + a.E * (a.pad - 1));
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(moe_score_kernel<float>, dim3(a.T), dim3(256), (size_t)a.E * 4, st, a)
                                        : launch_pdl(moe_score_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), (size_t)a.E * 4, st, a);
  KGE_CUDA_OK(ce);
  KGE_CUDA_OK(launch_pdl(moe_group_kernel, dim3(1), dim3(1024), (size_t)2 * a.E * 4, st, a));
  return 0;
}

}  // namespace kge
