// Recurrent token mixers with per-request state slots, in bfloat16 or float32 storage and fp32 state:
//   - the gated linear recurrence (RG-LRU): causal per-channel convolution whose last inputs are carried in the slot,
//     then S <- a S + sqrt(1 - a^2) i u with a = exp(-c r softplus(lam)), one thread per (request, channel);
//   - the matrix memory (mLSTM) with a running maximum that starts at 0, one block per (request, head), the dim x vdim
//     state in shared memory, one thread per value column.
// A request whose first row of the step is position 0 starts from zero; otherwise from what its slot holds.  Rows of a
// request are processed in order, so cutting a prompt into steps anywhere gives the same arithmetic.
#include <algorithm>

#include "common.cuh"
#include "elt_access.cuh"
#include "hybrid_ops.h"

namespace kge {

constexpr int MAX_TAPS = 16;

template <typename E>
__global__ void rglru_conv_kernel(RglruArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int b = a.token_req[t], pos = a.positions[t], rs = a.qsl[b];
  const int p0 = a.positions[rs];                         // position of the request's first row in this step
  const E* yx = (const E*)a.yx;
  const float* tail = a.state + (int64_t)a.slots[b] * a.slot_stride + a.width;
  for (int c = threadIdx.x; c < a.width; c += blockDim.x) {
    float acc = ldf((const E*)a.conv_b + c);
    for (int j = 0; j < a.taps; ++j) {
      const int back = a.taps - 1 - j, sp = pos - back;
      float xv = 0.f;
      if (sp >= p0) xv = ldf(yx + (int64_t)(t - back) * 2 * a.width + a.width + c);
      else if (sp >= 0) xv = tail[(int64_t)(sp - p0 + a.taps - 1) * a.width + c];
      acc = fmaf(ldf((const E*)a.conv_w + (int64_t)c * a.taps + j), xv, acc);
    }
    stf((E*)a.u + (int64_t)t * a.width + c, acc);
  }
}

int rglru_conv(const RglruArgs& a, cudaStream_t st) {
  if (a.T <= 0) return 0;
  KGE_REQUIRE(a.taps >= 1 && a.taps <= MAX_TAPS, "rglru_conv: %d taps (1..%d)", a.taps, MAX_TAPS);
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(rglru_conv_kernel<float>, dim3(a.T), dim3(256), 0, st, a)
                                        : launch_pdl(rglru_conv_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), 0, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

__device__ __forceinline__ float sigmoidf_(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ float softplusf_(float v) { return v > 20.f ? v : log1pf(expf(v)); }
__device__ __forceinline__ float gelu_tanhf_(float v) { return 0.5f * v * (1.f + tanhf(0.79788456080286536f * (v + 0.044715f * v * v * v))); }

template <typename E>
__global__ void __launch_bounds__(128) rglru_scan_kernel(RglruArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.width) return;
  const int rs = a.qsl[b], re = a.qsl[b + 1], p0 = a.positions[rs], n = re - rs;
  float* slot = a.state + (int64_t)a.slots[b] * a.slot_stride;
  const E* yx = (const E*)a.yx;
  const E* u = (const E*)a.u;
  E* out = (E*)a.out;
  const float sp = a.decay_c * softplusf_(ldf((const E*)a.lam + c));
  float S = p0 > 0 ? slot[c] : 0.f;
  // eight tokens at a time: all their operands are requested before the first is used, so the recurrence itself - one
  // dependent fma per token - is what the loop waits for, not a memory round trip per token
  constexpr int G = 8;
  for (int t0 = rs; t0 < re; t0 += G) {
    float gr[G], gi[G], uv[G], yv[G];
#pragma unroll
    for (int k = 0; k < G; ++k) {
      const int t = min(t0 + k, re - 1);
      gr[k] = a.gates[(int64_t)t * 2 * a.width + c];
      gi[k] = a.gates[(int64_t)t * 2 * a.width + a.width + c];
      uv[k] = ldf(u + (int64_t)t * a.width + c);
      yv[k] = ldf(yx + (int64_t)t * 2 * a.width + c);
    }
#pragma unroll
    for (int k = 0; k < G; ++k) {
      if (t0 + k < re) {
        const float r = sigmoidf_(gr[k]), i = sigmoidf_(gi[k]);
        const float log_a = -sp * r;
        const float av = expf(log_a);
        const float mult = sqrtf(-expm1f(2.f * log_a));          // sqrt(1 - a^2) without cancellation near a = 1
        S = fmaf(av, S, mult * i * uv[k]);
        stf(out + (int64_t)(t0 + k) * a.width + c, S * gelu_tanhf_(yv[k]));
      }
    }
  }
  slot[c] = S;
  // the conv's next inputs: positions p1 - (taps - 1) .. p1 - 1 with p1 = p0 + n, from this step's rows or the old tail
  float nt[MAX_TAPS];
  float* tail = slot + a.width;
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) {
    if (k >= a.taps - 1) break;
    const int sp2 = p0 + n - (a.taps - 1) + k;
    float v = 0.f;
    if (sp2 >= p0) v = ldf(yx + (int64_t)(rs + sp2 - p0) * 2 * a.width + a.width + c);
    else if (sp2 >= 0) v = tail[(int64_t)(sp2 - p0 + a.taps - 1) * a.width + c];
    nt[k] = v;
  }
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) {
    if (k >= a.taps - 1) break;
    tail[(int64_t)k * a.width + c] = nt[k];
  }
}

// Prompt steps: everything of the recurrence that does not depend on the previous token is done for all tokens at once.
// rglru_ab_kernel turns the gate pre-activations, in place, into the recurrence's coefficients (a_t, b_t = sqrt(1 - a_t^2)
// i_t u_t); rglru_chain_kernel is then one fma per token and channel (S_t written over a_t) plus the state hand-over; and
// rglru_out_kernel multiplies by gelu(y).  Same arithmetic per element as the fused kernel.
template <typename E>
__global__ void rglru_ab_kernel(RglruArgs a, float* gates) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n = (int64_t)a.T * a.width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / a.width; const int c = (int)(i % a.width);
    const float sp = a.decay_c * softplusf_(ldf((const E*)a.lam + c));
    const float r = sigmoidf_(gates[t * 2 * a.width + c]), ig = sigmoidf_(gates[t * 2 * a.width + a.width + c]);
    const float log_a = -sp * r;
    gates[t * 2 * a.width + c] = expf(log_a);
    gates[t * 2 * a.width + a.width + c] = sqrtf(-expm1f(2.f * log_a)) * ig * ldf((const E*)a.u + t * a.width + c);
  }
}

template <typename E>
__global__ void __launch_bounds__(128) rglru_chain_kernel(RglruArgs a, float* gates) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.width) return;
  const int rs = a.qsl[b], re = a.qsl[b + 1], p0 = a.positions[rs], n = re - rs;
  float* slot = a.state + (int64_t)a.slots[b] * a.slot_stride;
  const E* yx = (const E*)a.yx;
  float S = p0 > 0 ? slot[c] : 0.f;
  constexpr int G = 8;
  for (int t0 = rs; t0 < re; t0 += G) {
    float av[G], bv[G];
#pragma unroll
    for (int k = 0; k < G; ++k) {
      const int t = min(t0 + k, re - 1);
      av[k] = gates[(int64_t)t * 2 * a.width + c];
      bv[k] = gates[(int64_t)t * 2 * a.width + a.width + c];
    }
#pragma unroll
    for (int k = 0; k < G; ++k) {
      if (t0 + k < re) {
        S = fmaf(av[k], S, bv[k]);
        gates[(int64_t)(t0 + k) * 2 * a.width + c] = S;
      }
    }
  }
  slot[c] = S;
  float nt[MAX_TAPS];
  float* tail = slot + a.width;
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) {
    if (k >= a.taps - 1) break;
    const int sp2 = p0 + n - (a.taps - 1) + k;
    float v = 0.f;
    if (sp2 >= p0) v = ldf(yx + (int64_t)(rs + sp2 - p0) * 2 * a.width + a.width + c);
    else if (sp2 >= 0) v = tail[(int64_t)(sp2 - p0 + a.taps - 1) * a.width + c];
    nt[k] = v;
  }
#pragma unroll
  for (int k = 0; k < MAX_TAPS; ++k) {
    if (k >= a.taps - 1) break;
    tail[(int64_t)k * a.width + c] = nt[k];
  }
}

template <typename E>
__global__ void rglru_out_kernel(RglruArgs a, const float* gates) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n = (int64_t)a.T * a.width;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / a.width; const int c = (int)(i % a.width);
    stf((E*)a.out + i, gates[t * 2 * a.width + c] * gelu_tanhf_(ldf((const E*)a.yx + t * 2 * a.width + c)));
  }
}

int rglru_scan(const RglruArgs& a, cudaStream_t st) {
  if (a.T <= 0 || a.B <= 0) return 0;
  KGE_REQUIRE(a.taps >= 1 && a.taps <= MAX_TAPS, "rglru_scan: %d taps (1..%d)", a.taps, MAX_TAPS);
  const dim3 grid(a.B, (a.width + 127) / 128), block(128);
  if (a.T > a.B) {                       // some request brings several rows
    float* gates = const_cast<float*>(a.gates);
    const int eg = (int)std::min<int64_t>(((int64_t)a.T * a.width + 255) / 256, 148 * 16);
    if (a.elt == KGE_ELT_F32) {
      KGE_CUDA_OK(launch_pdl(rglru_ab_kernel<float>, dim3(eg), dim3(256), 0, st, a, gates));
      KGE_CUDA_OK(launch_pdl(rglru_chain_kernel<float>, grid, block, 0, st, a, gates));
      KGE_CUDA_OK(launch_pdl(rglru_out_kernel<float>, dim3(eg), dim3(256), 0, st, a, (const float*)gates));
    } else {
      KGE_CUDA_OK(launch_pdl(rglru_ab_kernel<__nv_bfloat16>, dim3(eg), dim3(256), 0, st, a, gates));
      KGE_CUDA_OK(launch_pdl(rglru_chain_kernel<__nv_bfloat16>, grid, block, 0, st, a, gates));
      KGE_CUDA_OK(launch_pdl(rglru_out_kernel<__nv_bfloat16>, dim3(eg), dim3(256), 0, st, a, (const float*)gates));
    }
    return 0;
  }
  cudaError_t ce = a.elt == KGE_ELT_F32 ? launch_pdl(rglru_scan_kernel<float>, grid, block, 0, st, a)
                                        : launch_pdl(rglru_scan_kernel<__nv_bfloat16>, grid, block, 0, st, a);
  KGE_CUDA_OK(ce);
  return 0;
}

// ------------------------------------------------------------------------------------------------ matrix memory
template <typename E>
__global__ void mlstm_step_kernel(MlstmArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int dim = a.dim, vdim = a.vdim;
  float* S = sm;                       // [dim][vdim]
  float* nv = S + (int64_t)dim * vdim; // [dim]
  float* ks = nv + dim;                // [dim]
  float* qs = ks + dim;                // [dim]
  float* red = qs + dim;               // [33]
  const int rs = a.qsl[b], re = a.qsl[b + 1], p0 = a.positions[rs];
  float* slot = a.state + (int64_t)a.slots[b] * a.slot_stride + (int64_t)h * ((int64_t)dim * vdim + dim + 1);
  const bool fresh = p0 == 0;
  for (int i = tid; i < dim * vdim + dim; i += blockDim.x) S[i] = fresh ? 0.f : slot[i];     // S then n: contiguous in both
  float m = fresh ? 0.f : slot[(int64_t)dim * vdim + dim];
  __syncthreads();
  const E *qp = (const E*)a.q, *kp = (const E*)a.k, *vp = (const E*)a.v, *gp = (const E*)a.g;
  const float nw = tid < vdim ? ldf((const E*)a.norm_w + h * vdim + tid) : 0.f;
  for (int t = rs; t < re; ++t) {
    if (tid < dim) {
      ks[tid] = ldf(kp + (int64_t)t * a.ld + h * dim + tid);
      qs[tid] = ldf(qp + (int64_t)t * a.ld + h * dim + tid) * a.q_scale;
    }
    const float ip = a.gates[(int64_t)t * 2 * a.H + h], fp = a.gates[(int64_t)t * 2 * a.H + a.H + h];
    const float it = a.cap * tanhf(ip / a.cap);
    const float fc = a.cap * tanhf(fp / a.cap);
    const float ft = fminf(fc, 0.f) - log1pf(expf(-fabsf(fc)));          // logsigmoid
    const float mn = fmaxf(ft + m, it);
    const float fa = expf(ft + m - mn), ia = expf(it - mn);
    m = mn;
    __syncthreads();
    float part = 0.f;
    if (tid < dim) {
      const float nn = fmaf(fa, nv[tid], ia * ks[tid]);
      nv[tid] = nn;
      part = nn * qs[tid];
    }
    const float nq = block_sum(part, red);
    float o = 0.f;
    if (tid < vdim) {
      const float vv = ia * ldf(vp + (int64_t)t * a.ld + h * vdim + tid);
      float num = 0.f;
      for (int d = 0; d < dim; ++d) {
        const float s = fmaf(fa, S[d * vdim + tid], ks[d] * vv);
        S[d * vdim + tid] = s;
        num = fmaf(s, qs[d], num);
      }
      o = num / (fmaxf(fabsf(nq), expf(-m)) + a.den_eps);
    }
    const float ss = block_sum(o * o, red);
    if (tid < vdim) {
      const float inv = 1.f / sqrtf(ss / (float)vdim + a.eps);
      const float gate = 1.f / (1.f + expf(-ldf(gp + (int64_t)t * a.ld + h * vdim + tid)));
      stf((E*)a.out + (int64_t)t * a.ldo + h * vdim + tid, o * inv * nw * gate * a.out_scale);
    }
  }
  __syncthreads();
  for (int i = tid; i < dim * vdim + dim; i += blockDim.x) slot[i] = S[i];
  if (tid == 0) slot[(int64_t)dim * vdim + dim] = m;
}

// The same recurrence with a head's value columns split over blocks of 64 threads: a thread keeps its column of the
// state in registers (dim <= 128), the first warp keeps the normaliser n, and the un-normalised read-out goes to an fp32
// scratch; mlstm_norm_gate_kernel then divides each head by its root mean square and applies weight and output gate.
// More blocks than (request, head) pairs fill the machine when few requests prefill, and the state never sits in shared memory.
constexpr int ML_MAXD = 128, ML_COLS = 64, ML_THREADS = ML_COLS + 32;      // two warps of value columns, one for the normaliser

// gate pre-activations -> log gates, in place, for every token at once (the recurrence then needs two exponentials a token)
__global__ void mlstm_log_gates_kernel(float* gates, int T, int H, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * 2 * H) return;
  const float c = cap * tanhf(gates[i] / cap);
  gates[i] = (i % (2 * H)) < H ? c : fminf(c, 0.f) - log1pf(expf(-fabsf(c)));     // input gate | logsigmoid for the forget gate
}

template <typename E>
__global__ void __launch_bounds__(ML_THREADS) mlstm_cols_kernel(MlstmArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) float ks[ML_MAXD], qs[ML_MAXD], nv[ML_MAXD];
  __shared__ float nq_s;
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, c = blockIdx.z * ML_COLS + tid;
  const int dim = a.dim, vdim = a.vdim;
  const bool colw = tid < ML_COLS;                 // a value-column thread (the last warp keeps n instead)
  const bool col = colw && c < vdim;
  const int rs = a.qsl[b], re = a.qsl[b + 1], p0 = a.positions[rs];
  float* slot = a.state + (int64_t)a.slots[b] * a.slot_stride + (int64_t)h * ((int64_t)dim * vdim + dim + 1);
  const bool fresh = p0 == 0;
  float S[ML_MAXD];
#pragma unroll
  for (int d = 0; d < ML_MAXD; ++d) S[d] = (d < dim && col && !fresh) ? slot[(int64_t)d * vdim + c] : 0.f;
  for (int d = tid; d < ML_MAXD; d += ML_THREADS) { nv[d] = (d < dim && !fresh) ? slot[(int64_t)dim * vdim + d] : 0.f; ks[d] = 0.f; qs[d] = 0.f; }
  float m = fresh ? 0.f : slot[(int64_t)dim * vdim + dim];
  const E *qp = (const E*)a.q, *kp = (const E*)a.k, *vp = (const E*)a.v;
  __syncthreads();
  // operands of the NEXT token are requested while the current one is computed (two key / query entries per thread)
  float kn[2], qn[2], vn, ipn, fpn;
  auto fetch = [&](int t) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int d = tid + j * ML_COLS;
      kn[j] = (colw && d < dim) ? ldf(kp + (int64_t)t * a.ld + h * dim + d) : 0.f;
      qn[j] = (colw && d < dim) ? ldf(qp + (int64_t)t * a.ld + h * dim + d) * a.q_scale : 0.f;
    }
    vn = col ? ldf(vp + (int64_t)t * a.ld + h * vdim + c) : 0.f;
    ipn = a.gates[(int64_t)t * 2 * a.H + h];
    fpn = a.gates[(int64_t)t * 2 * a.H + a.H + h];
  };
  if (rs < re) fetch(rs);
  for (int t = rs; t < re; ++t) {
    if (colw) { ks[tid] = kn[0]; ks[tid + ML_COLS] = kn[1]; qs[tid] = qn[0]; qs[tid + ML_COLS] = qn[1]; }
    const float it = ipn, ft = fpn, vcur = vn;     // log gates (mlstm_log_gates_kernel ran before)
    if (t + 1 < re) fetch(t + 1);
    const float mn = fmaxf(ft + m, it);
    const float fa = expf(ft + m - mn), ia = expf(it - mn);
    m = mn;
    const float vv = ia * vcur;
    __syncthreads();
    float num = 0.f;
    if (!colw) {
      const int ln = tid - ML_COLS;
      float part = 0.f;
      for (int d = ln; d < dim; d += 32) {
        const float nn = fmaf(fa, nv[d], ia * ks[d]);
        nv[d] = nn;
        part = fmaf(nn, qs[d], part);
      }
      part = warp_sum(part);
      if (ln == 0) nq_s = part;
    } else {
      float n0 = 0.f, n1 = 0.f, n2 = 0.f, n3 = 0.f;       // four chains: the read-out does not wait on one long dependency
#pragma unroll
      for (int d4 = 0; d4 < ML_MAXD / 4; ++d4) {
        if (d4 * 4 < dim) {                      // dim is a multiple of 4 on this path
          const float4 k4 = reinterpret_cast<const float4*>(ks)[d4], q4 = reinterpret_cast<const float4*>(qs)[d4];
          S[d4 * 4 + 0] = fmaf(fa, S[d4 * 4 + 0], k4.x * vv); n0 = fmaf(S[d4 * 4 + 0], q4.x, n0);
          S[d4 * 4 + 1] = fmaf(fa, S[d4 * 4 + 1], k4.y * vv); n1 = fmaf(S[d4 * 4 + 1], q4.y, n1);
          S[d4 * 4 + 2] = fmaf(fa, S[d4 * 4 + 2], k4.z * vv); n2 = fmaf(S[d4 * 4 + 2], q4.z, n2);
          S[d4 * 4 + 3] = fmaf(fa, S[d4 * 4 + 3], k4.w * vv); n3 = fmaf(S[d4 * 4 + 3], q4.w, n3);
        }
      }
      num = (n0 + n1) + (n2 + n3);
    }
    __syncthreads();
    if (col) a.o_scratch[(int64_t)t * a.H * vdim + h * vdim + c] = num / (fmaxf(fabsf(nq_s), expf(-m)) + a.den_eps);
  }
  if (col) {
#pragma unroll
    for (int d = 0; d < ML_MAXD; ++d) if (d < dim) slot[(int64_t)d * vdim + c] = S[d];
  }
  if (blockIdx.z == 0) {
    __syncthreads();
    for (int d = tid; d < dim; d += ML_THREADS) slot[(int64_t)dim * vdim + d] = nv[d];
    if (tid == 0) slot[(int64_t)dim * vdim + dim] = m;
  }
}

// Prompts: the same recurrence evaluated 32 tokens at a time (chunkwise form), all in fp32.  With b_t the running sum of
// the log forget gates inside the chunk and (C, n, m) the state before it,
//   m_t = max(b_t + m, max_{s<=t}(b_t - b_s + i_s))                     (equal to the step-by-step maximum)
//   num_t = e^(b_t + m - m_t) C^T q_t + sum_{s<=t} e^(b_t - b_s + i_s - m_t) (q_t . k_s) v_s
//   n_t . q_t likewise with n and the same weights;   C' = e^(b_L + m - m_L) C + sum_s e^(b_L - b_s + i_s - m_L) k_s v_s^T
// so a token costs the same multiply-adds as one recurrence step but the 32 tokens of a chunk are independent: no
// barrier and no dependent chain per token.  A thread still owns one value column of C in registers.
constexpr int ML_CH = 32, ML_NSL = 4, ML_DS = ML_MAXD / ML_NSL;      // tokens per chunk; key-dimension slices per column; dims per slice
constexpr int MC_COLS = 32;          // value columns per block of the chunkwise kernel: more, smaller blocks fill the machine when few requests prefill

// Block = 32 value columns x 4 slices of the key dimension (128 threads): a thread keeps C[its 32 dims][its column] in
// registers, so the read-out and the update of a chunk are spread over four warps; the slices' partial read-outs meet in
// shared memory and are summed in slice order.
template <typename E>
__global__ void __launch_bounds__(MC_COLS * ML_NSL) mlstm_chunk_kernel(MlstmArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float csm[];
  constexpr int NT = MC_COLS * ML_NSL;
  const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, ct = tid % MC_COLS, sl = tid / MC_COLS, c = blockIdx.z * MC_COLS + ct;
  const int dim = a.dim, vdim = a.vdim, d0 = sl * ML_DS;
  float* qs = csm;                           // [ML_CH][dim]   q_t * q_scale
  float* ks = qs + ML_CH * dim;              // [ML_CH][dim]   k_s, later u_s * k_s
  float* Sw = ks + ML_CH * dim;              // [ML_CH][ML_CH] weighted scores (s <= t)
  float* nv = Sw + ML_CH * ML_CH;            // [ML_MAXD]
  float* li = nv + ML_MAXD;                  // [ML_CH] log input gate
  float* bc = li + ML_CH;                    // [ML_CH] running sum of log forget gates
  float* mt = bc + ML_CH;                    // [ML_CH] running maximum
  float* nq = mt + ML_CH;                    // [ML_CH] n . q_t (state part)
  float* us = nq + ML_CH;                    // [ML_CH] weight of token s in the state after the chunk
  float* vs = us + ML_CH;                    // [ML_CH][MC_COLS] this block's value columns of the chunk's tokens
  float* part = vs + ML_CH * MC_COLS;        // [ML_NSL][ML_CH][MC_COLS] partial read-outs of the slices
  const bool col = c < vdim;
  const int rs = a.qsl[b], re = a.qsl[b + 1], p0 = a.positions[rs];
  float* slot = a.state + (int64_t)a.slots[b] * a.slot_stride + (int64_t)h * ((int64_t)dim * vdim + dim + 1);
  const bool fresh = p0 == 0;
  float C[ML_DS];
#pragma unroll
  for (int d = 0; d < ML_DS; ++d) C[d] = (d0 + d < dim && col && !fresh) ? slot[(int64_t)(d0 + d) * vdim + c] : 0.f;
  for (int d = tid; d < ML_MAXD; d += NT) nv[d] = (d < dim && !fresh) ? slot[(int64_t)dim * vdim + d] : 0.f;
  float m = fresh ? 0.f : slot[(int64_t)dim * vdim + dim];
  const E *qp = (const E*)a.q, *kp = (const E*)a.k, *vp = (const E*)a.v;
  for (int t0 = rs; t0 < re; t0 += ML_CH) {
    const int L = min(ML_CH, re - t0);
    __syncthreads();                                         // the previous chunk's shared arrays are no longer read
    for (int i = tid; i < L * dim; i += NT) {
      const int t = i / dim, d = i % dim;
      qs[i] = ldf(qp + (int64_t)(t0 + t) * a.ld + h * dim + d) * a.q_scale;
      ks[i] = ldf(kp + (int64_t)(t0 + t) * a.ld + h * dim + d);
    }
    for (int i = tid; i < L * MC_COLS; i += NT) {
      const int s2 = i / MC_COLS, cc = blockIdx.z * MC_COLS + i % MC_COLS;
      vs[i] = cc < vdim ? ldf(vp + (int64_t)(t0 + s2) * a.ld + h * vdim + cc) : 0.f;
    }
    if (tid == 0) {                                          // the chunk's gate scalars: 32 short steps
      float run = 0.f, mm = m;
      for (int t = 0; t < L; ++t) {
        const float it = a.gates[(int64_t)(t0 + t) * 2 * a.H + h], ft = a.gates[(int64_t)(t0 + t) * 2 * a.H + a.H + h];
        mm = fmaxf(ft + mm, it);
        run += ft;
        li[t] = it; bc[t] = run; mt[t] = mm;
      }
    }
    __syncthreads();
    const float bL = bc[L - 1], mL = mt[L - 1];
    // weighted scores Sw[t][s] = e^(b_t - b_s + i_s - m_t) (q_t . k_s) for s <= t; the state part of n . q_t; the tokens' weights in the new state
    for (int i = tid; i < L * L; i += NT) {
      const int t = i / L, s2 = i % L;
      float w = 0.f;
      if (s2 <= t) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (int d4 = 0; d4 < dim / 4; ++d4) {
          const float4 q4 = reinterpret_cast<const float4*>(qs + t * dim)[d4], k4 = reinterpret_cast<const float4*>(ks + s2 * dim)[d4];
          a0 = fmaf(q4.x, k4.x, a0); a1 = fmaf(q4.y, k4.y, a1); a2 = fmaf(q4.z, k4.z, a2); a3 = fmaf(q4.w, k4.w, a3);
        }
        w = expf(bc[t] - bc[s2] + li[s2] - mt[t]) * ((a0 + a1) + (a2 + a3));
      }
      Sw[t * ML_CH + s2] = w;
    }
    for (int t = tid; t < L; t += NT) {
      float acc = 0.f;
      for (int d = 0; d < dim; ++d) acc = fmaf(nv[d], qs[t * dim + d], acc);
      nq[t] = acc;
      us[t] = expf(bL - bc[t] + li[t] - mL);
    }
    // this slice's part of C^T q_t for every token of the chunk
    for (int t = 0; t < L; ++t) {
      float n0 = 0.f, n1 = 0.f, n2 = 0.f, n3 = 0.f;
#pragma unroll
      for (int d4 = 0; d4 < ML_DS / 4; ++d4) {
        if (d0 + d4 * 4 < dim) {
          const float4 q4 = reinterpret_cast<const float4*>(qs + t * dim + d0)[d4];
          n0 = fmaf(C[d4 * 4 + 0], q4.x, n0); n1 = fmaf(C[d4 * 4 + 1], q4.y, n1);
          n2 = fmaf(C[d4 * 4 + 2], q4.z, n2); n3 = fmaf(C[d4 * 4 + 3], q4.w, n3);
        }
      }
      part[(sl * ML_CH + t) * MC_COLS + ct] = (n0 + n1) + (n2 + n3);
    }
    __syncthreads();
    // tokens t = sl, sl + 4, ...: slices summed in order, the chunk's own tokens added, normaliser, out
    for (int t = sl; t < L; t += ML_NSL) {
      float inter = 0.f;
#pragma unroll
      for (int k = 0; k < ML_NSL; ++k) inter += part[(k * ML_CH + t) * MC_COLS + ct];
      float intra = 0.f, rowsum = 0.f;
      for (int s2 = 0; s2 <= t; ++s2) { const float w = Sw[t * ML_CH + s2]; intra = fmaf(w, vs[s2 * MC_COLS + ct], intra); rowsum += w; }
      const float g = expf(bc[t] + m - mt[t]);
      const float num = fmaf(g, inter, intra);
      const float den = fmaxf(fabsf(fmaf(g, nq[t], rowsum)), expf(-mt[t])) + a.den_eps;
      if (col) a.o_scratch[(int64_t)(t0 + t) * a.H * vdim + h * vdim + c] = num / den;
    }
    // state after the chunk: C' = G C + sum_s u_s k_s v_s^T with G = e^(b_L + m - m_L); n likewise
    const float G = expf(bL + m - mL);
#pragma unroll
    for (int d = 0; d < ML_DS; ++d) C[d] *= G;
    for (int s2 = 0; s2 < L; ++s2) {
      const float x = us[s2] * vs[s2 * MC_COLS + ct];
#pragma unroll
      for (int d4 = 0; d4 < ML_DS / 4; ++d4) {
        if (d0 + d4 * 4 < dim) {
          const float4 k4 = reinterpret_cast<const float4*>(ks + s2 * dim + d0)[d4];
          C[d4 * 4 + 0] = fmaf(k4.x, x, C[d4 * 4 + 0]); C[d4 * 4 + 1] = fmaf(k4.y, x, C[d4 * 4 + 1]);
          C[d4 * 4 + 2] = fmaf(k4.z, x, C[d4 * 4 + 2]); C[d4 * 4 + 3] = fmaf(k4.w, x, C[d4 * 4 + 3]);
        }
      }
    }
    for (int d = tid; d < dim; d += NT) {
      float acc = G * nv[d];
      for (int s2 = 0; s2 < L; ++s2) acc = fmaf(us[s2], ks[s2 * dim + d], acc);
      nv[d] = acc;
    }
    m = mL;
  }
  __syncthreads();
  if (col) {
#pragma unroll
    for (int d = 0; d < ML_DS; ++d) if (d0 + d < dim) slot[(int64_t)(d0 + d) * vdim + c] = C[d];
  }
  if (blockIdx.z == 0) {
    for (int d = tid; d < dim; d += NT) slot[(int64_t)dim * vdim + d] = nv[d];
    if (tid == 0) slot[(int64_t)dim * vdim + dim] = m;
  }
}

template <typename E>
__global__ void mlstm_norm_gate_kernel(MlstmArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x, h = blockIdx.y;
  const float* o = a.o_scratch + (int64_t)t * a.H * a.vdim + h * a.vdim;
  float ss = 0.f;
  for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) ss = fmaf(o[c], o[c], ss);
  ss = block_sum(ss, red);
  const float inv = a.out_scale / sqrtf(ss / (float)a.vdim + a.eps);
  for (int c = threadIdx.x; c < a.vdim; c += blockDim.x) {
    const float gate = 1.f / (1.f + expf(-ldf((const E*)a.g + (int64_t)t * a.ld + h * a.vdim + c)));
    stf((E*)a.out + (int64_t)t * a.ldo + h * a.vdim + c, o[c] * inv * ldf((const E*)a.norm_w + h * a.vdim + c) * gate);
  }
}

int mlstm_step(const MlstmArgs& a, cudaStream_t st) {
  if (a.T <= 0 || a.B <= 0) return 0;
  if (a.o_scratch && a.dim <= ML_MAXD && a.dim % 4 == 0 && a.H <= 65535) {
    const dim3 grid(a.B, a.H, (a.vdim + ML_COLS - 1) / ML_COLS), g2(a.T, a.H);
    const int nt = std::min(256, (a.vdim + 31) / 32 * 32);
    KGE_CUDA_OK(launch_pdl(mlstm_log_gates_kernel, dim3((a.T * 2 * a.H + 255) / 256), dim3(256), 0, st, const_cast<float*>(a.gates), a.T, a.H, a.cap));
    const size_t csm_bytes = ((size_t)2 * ML_CH * a.dim + ML_CH * ML_CH + ML_MAXD + 5 * ML_CH + (1 + ML_NSL) * ML_CH * MC_COLS) * 4;
    const dim3 cgrid(a.B, a.H, (a.vdim + MC_COLS - 1) / MC_COLS);
    if (a.T > a.B) {
      // some request brings several rows: 32 tokens at a time (single-token requests of the same step are chunks of one)
      static bool smem_set = false;
      if (!smem_set) {
        KGE_CUDA_OK(cudaFuncSetAttribute(mlstm_chunk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        KGE_CUDA_OK(cudaFuncSetAttribute(mlstm_chunk_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        smem_set = true;
      }
      if (a.elt == KGE_ELT_F32) KGE_CUDA_OK(launch_pdl(mlstm_chunk_kernel<float>, cgrid, dim3(MC_COLS * ML_NSL), csm_bytes, st, a));
      else KGE_CUDA_OK(launch_pdl(mlstm_chunk_kernel<__nv_bfloat16>, cgrid, dim3(MC_COLS * ML_NSL), csm_bytes, st, a));
      if (a.elt == KGE_ELT_F32) KGE_CUDA_OK(launch_pdl(mlstm_norm_gate_kernel<float>, g2, dim3(nt), 0, st, a));
      else KGE_CUDA_OK(launch_pdl(mlstm_norm_gate_kernel<__nv_bfloat16>, g2, dim3(nt), 0, st, a));
      return 0;
    }
    if (a.elt == KGE_ELT_F32) {
      KGE_CUDA_OK(launch_pdl(mlstm_cols_kernel<float>, grid, dim3(ML_THREADS), 0, st, a));
      KGE_CUDA_OK(launch_pdl(mlstm_norm_gate_kernel<float>, g2, dim3(nt), 0, st, a));
    } else {
      KGE_CUDA_OK(launch_pdl(mlstm_cols_kernel<__nv_bfloat16>, grid, dim3(ML_THREADS), 0, st, a));
      KGE_CUDA_OK(launch_pdl(mlstm_norm_gate_kernel<__nv_bfloat16>, g2, dim3(nt), 0, st, a));
    }
    return 0;
  }
  const int threads = (std::max(a.dim, a.vdim) + 31) / 32 * 32;
  KGE_REQUIRE(threads <= 1024, "mlstm_step: head sizes %d x %d need more than 1024 threads", a.dim, a.vdim);
  const size_t smem = ((size_t)a.dim * a.vdim + 3 * (size_t)a.dim + 64) * 4;
  KGE_REQUIRE(smem <= 227 * 1024, "mlstm_step: a %d x %d state does not fit shared memory", a.dim, a.vdim);
  const dim3 grid(a.B, a.H), block(threads);
  cudaError_t ce;
  if (a.elt == KGE_ELT_F32) {
    cudaFuncSetAttribute(mlstm_step_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ce = launch_pdl(mlstm_step_kernel<float>, grid, block, smem, st, a);
  } else {
    cudaFuncSetAttribute(mlstm_step_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ce = launch_pdl(mlstm_step_kernel<__nv_bfloat16>, grid, block, smem, st, a);
  }
  KGE_CUDA_OK(ce);
  return 0;
}

}  // namespace kge
