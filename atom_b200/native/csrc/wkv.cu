// Linear recurrence with a decay per key channel and a bonus for the present token, per request and head:
//   o_t[j] = sum_i r_t[i] * (S[i][j] + u[i] * k_t[i] * v_t[j])
//   S[i][j] <- w_t[i] * S[i][j] + k_t[i] * v_t[j],        w_t[i] = exp(-exp(d_t[i] + w0[i]))
// followed by what the mixer does with o before its output product: each head's o divided by its root
// mean square, times a weight per channel, times silu(gate).  The state S [dk, dv] is 32-bit, lives in
// the request's state row between steps, and all arithmetic of the recurrence is 32-bit; r, k, v, d and
// the gate come from matrix products in the activation type.
//
// One block per (request, head); a state column j (the columns do not depend on one another) belongs to
// SPLIT (8 or 4) neighbouring lanes, each of which keeps its share of the column's key channels in registers, so
// a token costs dk / SPLIT multiply-adds per thread and log2 SPLIT shuffles, and the token-to-token chain is short.
// The bonus needs no pass over the state: sum_i r[i] u[i] k[i] v[j] = v[j] * b with one number b per token,
// which is formed while the chunk is staged.  Tokens go through shared memory in chunks of up to 32: r, k and
// the decay of a chunk are converted (and the two exponentials taken) once, by all threads; the next chunk's
// inputs are already on their way into registers while the present chunk runs, since with one CTA per
// (request, head) nothing else would hide the round trips to memory.  The order of the sums does not depend on
// how a request's tokens are cut into steps or chunks.
#include "common.cuh"

namespace atom {

constexpr int kWkvChunk = 32;     // most tokens staged at a time
constexpr int kWkvRegs = 8;       // elements of each staged array that a thread holds in flight

// What a thread holds of the next chunk while the present one runs: the loads are issued before the
// recurrence and used after it, so their round trips to memory hide behind it.
template <typename T>
struct WkvStage {
  T r[kWkvRegs], k[kWkvRegs], v[kWkvRegs], g[kWkvRegs];
  float d[kWkvRegs];
};

// TOK consecutive tokens of one state column's share of channels: all loads stand before the stores, so the
// tokens' chains overlap (only S runs from token to token, one multiply-add each).  A lane's channels are the
// float4 groups part, part + SPLIT, part + 2 SPLIT, ...: the lanes of a column read consecutive bytes.
template <int TOK, int DKP, int SPLIT>
__device__ __forceinline__ void wkv_tokens(float (&S)[DKP / SPLIT], const float* __restrict__ r_s,
                                           const float* __restrict__ k_s, const float* __restrict__ w_s,
                                           const float* __restrict__ v_s, const float* __restrict__ b_s,
                                           float* __restrict__ o_s, int c, int dv, int j, int part, unsigned group_mask) {
  constexpr int DKQ = DKP / SPLIT;
  float vj[TOK], acc[TOK][2];
#pragma unroll
  for (int t = 0; t < TOK; ++t) {
    vj[t] = v_s[(c + t) * dv + j];
    acc[t][0] = 0.f;
    acc[t][1] = 0.f;
  }
#pragma unroll
  for (int m = 0; m < DKQ / 4; ++m) {
    float4 r4[TOK], k4[TOK], w4[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      const int at = (c + t) * DKP + (SPLIT * m + part) * 4;
      r4[t] = *reinterpret_cast<const float4*>(r_s + at);
      k4[t] = *reinterpret_cast<const float4*>(k_s + at);
      w4[t] = *reinterpret_cast<const float4*>(w_s + at);
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
      acc[t][0] = fmaf(r4[t].x, S[4 * m], acc[t][0]);
      acc[t][1] = fmaf(r4[t].y, S[4 * m + 1], acc[t][1]);
      acc[t][0] = fmaf(r4[t].z, S[4 * m + 2], acc[t][0]);
      acc[t][1] = fmaf(r4[t].w, S[4 * m + 3], acc[t][1]);
      S[4 * m] = fmaf(w4[t].x, S[4 * m], k4[t].x * vj[t]);
      S[4 * m + 1] = fmaf(w4[t].y, S[4 * m + 1], k4[t].y * vj[t]);
      S[4 * m + 2] = fmaf(w4[t].z, S[4 * m + 2], k4[t].z * vj[t]);
      S[4 * m + 3] = fmaf(w4[t].w, S[4 * m + 3], k4[t].w * vj[t]);
    }
  }
  float sum[TOK];
#pragma unroll
  for (int t = 0; t < TOK; ++t) sum[t] = acc[t][0] + acc[t][1];
#pragma unroll
  for (int o = 1; o < SPLIT; o <<= 1)                             // (a column's lanes are neighbours in one warp)
#pragma unroll
    for (int t = 0; t < TOK; ++t) sum[t] += __shfl_xor_sync(group_mask, sum[t], o);
  if (part == 0) {
#pragma unroll
    for (int t = 0; t < TOK; ++t) o_s[(c + t) * dv + j] = fmaf(b_s[c + t], vj[t], sum[t]);
  }
}

template <typename T, int DKP, int SPLIT>
__global__ void __launch_bounds__(512)
wkv_kernel(T* __restrict__ y, const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
           const void* __restrict__ d, int d_dtype, const T* __restrict__ gate, const void* __restrict__ w0,
           const void* __restrict__ u, const void* __restrict__ norm_w, int vec_dtype, float* __restrict__ state,
           const int* __restrict__ cu_q, const int* __restrict__ state_slots, int heads, int dk, int dv,
           float eps, int write_state, int chunk) {
  atom::pdl_trigger();
  atom::pdl_wait();
  constexpr int DKQ = DKP / SPLIT;        // channels per lane (a multiple of 4)
  extern __shared__ __align__(16) float smem[];
  float* r_s = smem;                          // [chunk][DKP]
  float* k_s = r_s + chunk * DKP;             // [chunk][DKP]
  float* w_s = k_s + chunk * DKP;             // [chunk][DKP]
  float* u_s = w_s + chunk * DKP;             // [DKP]
  float* w0_s = u_s + DKP;                    // [DKP]
  float* v_s = w0_s + DKP;                    // [chunk][dv]
  float* o_s = v_s + chunk * dv;              // [chunk][dv]
  float* g_s = o_s + chunk * dv;              // [chunk][dv] silu(gate)
  __shared__ float rstd_s[kWkvChunk];
  __shared__ float b_s[kWkvChunk];

  const int s = blockIdx.x, hd = blockIdx.y;
  const int t0 = cu_q[s], t1 = cu_q[s + 1];
  if (t1 <= t0) return;                       // a request without tokens in this step (padding)
  const int j = threadIdx.x / SPLIT, part = threadIdx.x % SPLIT;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int64_t ldk = (int64_t)heads * dk, ldv = (int64_t)heads * dv;
  float* S_g = state + (((int64_t)state_slots[s] * heads + hd) * dk) * dv;

  for (int i = threadIdx.x; i < DKP; i += blockDim.x) {
    u_s[i] = i < dk ? load_as_float(u, vec_dtype, (int64_t)hd * dk + i) : 0.f;
    w0_s[i] = i < dk ? load_as_float(w0, vec_dtype, (int64_t)hd * dk + i) : 0.f;
  }
  float S[DKQ];
#pragma unroll
  for (int i = 0; i < DKQ; ++i) {
    const int ch = ((i / 4) * SPLIT + part) * 4 + (i % 4);        // the channel that S[i] stands for
    S[i] = (ch < dk && j < dv) ? S_g[(int64_t)ch * dv + j] : 0.f;
  }

  WkvStage<T> st;
  auto fetch = [&](int c0, int n) {           // the chunk's inputs, from memory into registers
#pragma unroll
    for (int q = 0; q < kWkvRegs; ++q) {
      const int e = threadIdx.x + q * blockDim.x;
      const int c = e / DKP, i = e - c * DKP;
      if (e < n * DKP && i < dk) {
        const int64_t off = (int64_t)(c0 + c) * ldk + (int64_t)hd * dk + i;
        st.r[q] = r[off];
        st.k[q] = k[off];
        st.d[q] = load_as_float(d, d_dtype, off);
      }
      const int cv = e / dv, jj = e - cv * dv;
      if (e < n * dv) {
        const int64_t off = (int64_t)(c0 + cv) * ldv + (int64_t)hd * dv + jj;
        st.v[q] = v[off];
        st.g[q] = gate[off];
      }
    }
  };
  fetch(t0, min(chunk, t1 - t0));
  __syncthreads();

  for (int c0 = t0; c0 < t1; c0 += chunk) {
    const int n = min(chunk, t1 - c0);
    // registers -> shared memory, with the decay's two exponentials and the gate's silu taken here
#pragma unroll
    for (int q = 0; q < kWkvRegs; ++q) {
      const int e = threadIdx.x + q * blockDim.x;
      const int c = e / DKP, i = e - c * DKP;
      if (e < n * DKP) {
        const bool in = i < dk;
        r_s[e] = in ? to_float(st.r[q]) : 0.f;
        k_s[e] = in ? to_float(st.k[q]) : 0.f;
        w_s[e] = in ? expf(-expf(st.d[q] + w0_s[i])) : 1.f;
      }
      if (e < n * dv) {
        v_s[e] = to_float(st.v[q]);
        const float g = to_float(st.g[q]);
        g_s[e] = g / (1.f + expf(-g));
      }
    }
    __syncthreads();
    if (c0 + chunk < t1) fetch(c0 + chunk, min(chunk, t1 - c0 - chunk));       // in flight while this chunk runs
    // the bonus' number of every token: a warp per token, lanes stride over the channels
    for (int c = warp; c < n; c += nwarps) {
      float b = 0.f;
      for (int i = lane; i < DKP; i += 32) b = fmaf(r_s[c * DKP + i] * u_s[i], k_s[c * DKP + i], b);
      b = warp_sum(b);
      if (lane == 0) b_s[c] = b;
    }
    __syncthreads();
    if (j < dv) {
      const unsigned group_mask = ((1u << SPLIT) - 1u) << (lane & ~(SPLIT - 1));
      int c = 0;
      for (; c + 4 <= n; c += 4) wkv_tokens<4, DKP, SPLIT>(S, r_s, k_s, w_s, v_s, b_s, o_s, c, dv, j, part, group_mask);
      for (; c < n; ++c) wkv_tokens<1, DKP, SPLIT>(S, r_s, k_s, w_s, v_s, b_s, o_s, c, dv, j, part, group_mask);
    }
    __syncthreads();
    // each head's o over its root mean square: a warp per token
    for (int c = warp; c < n; c += nwarps) {
      float ss = 0.f;
      for (int jj = lane; jj < dv; jj += 32) ss = fmaf(o_s[c * dv + jj], o_s[c * dv + jj], ss);
      ss = warp_sum(ss);
      if (lane == 0) rstd_s[c] = rsqrtf(ss / (float)dv + eps);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n * dv; e += blockDim.x) {
      const int c = e / dv, jj = e - c * dv;
      const int64_t off = (int64_t)(c0 + c) * ldv + (int64_t)hd * dv + jj;
      y[off] = from_float<T>(o_s[e] * rstd_s[c] * load_as_float(norm_w, vec_dtype, (int64_t)hd * dv + jj) * g_s[e]);
    }
    __syncthreads();
  }
  if (write_state && j < dv) {
#pragma unroll
    for (int i = 0; i < DKQ; ++i) {
      const int ch = ((i / 4) * SPLIT + part) * 4 + (i % 4);
      if (ch < dk) S_g[(int64_t)ch * dv + j] = S[i];
    }
  }
}

template <typename T>
static int launch_wkv(T* y, const T* r, const T* k, const T* v, const void* d, int d_dtype, const T* gate,
                      const void* w0, const void* u, const void* norm_w, int vec_dtype, float* state,
                      const int* cu_q, const int* state_slots, int S, int heads, int dk, int dv, float eps,
                      int write_state, cudaStream_t stream) {
  // eight lanes to a state column where that stays within 512 threads (more warps to hide the token-to-token
  // latency behind, fewer channels per lane), else four
  const int split = dv <= 64 ? 8 : 4;
  const int threads = ((dv * split + 31) / 32) * 32;
  const int dkp = ((dk + 4 * split - 1) / (4 * split)) * (4 * split);
  // as many tokens at a time as a thread's registers hold of every staged array
  int chunk = kWkvRegs * threads / (dkp > dv ? dkp : dv);
  chunk = chunk > kWkvChunk ? kWkvChunk : chunk;
  if (chunk < 1) return ATOM_ERR_ARG;
  const size_t smem = sizeof(float) * ((size_t)3 * chunk * dkp + 2 * dkp + (size_t)3 * chunk * dv);
#define ATOM_WKV_CASE(N, SP)                                                                                       \
  if (dkp == N && split == SP) {                                                                                   \
    if (smem > 48 * 1024)                                                                                          \
      cudaFuncSetAttribute(wkv_kernel<T, N, SP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
    launch_pdl(wkv_kernel<T, N, SP>, dim3(S, heads), dim3(threads), smem, stream, y, r, k, v, d, d_dtype, gate,   \
               w0, u, norm_w, vec_dtype, state, cu_q, state_slots, heads, dk, dv, eps, write_state, chunk);        \
    return check_launch();                                                                                         \
  }
  ATOM_WKV_CASE(32, 8)
  ATOM_WKV_CASE(64, 8)
  ATOM_WKV_CASE(96, 8)
  ATOM_WKV_CASE(128, 8)
  ATOM_WKV_CASE(16, 4)
  ATOM_WKV_CASE(32, 4)
  ATOM_WKV_CASE(48, 4)
  ATOM_WKV_CASE(64, 4)
  ATOM_WKV_CASE(80, 4)
  ATOM_WKV_CASE(96, 4)
  ATOM_WKV_CASE(112, 4)
  ATOM_WKV_CASE(128, 4)
#undef ATOM_WKV_CASE
  return ATOM_ERR_ARG;
}

}  // namespace atom

// y, gate: [T, heads * dv]; r, k, d: [T, heads * dk]; v: [T, heads * dv]; w0, u: [heads * dk]; norm_w: [heads * dv]
// (all three of one type); state: [slots, heads, dk, dv] float32.  d may be float32 beside bf16 activations.
ATOM_EXPORT int atom_wkv(void* y, const void* r, const void* k, const void* v, int dtype, const void* d, int d_dtype,
                         const void* gate, const void* w0, const void* u, const void* norm_w, int vec_dtype,
                         float* state, const int* cu_q, const int* state_slots, int S, int heads, int dk, int dv,
                         float eps, int write_state, cudaStream_t stream) {
  if (S <= 0) return ATOM_OK;
  if (heads <= 0 || heads > 65535 || dk <= 0 || dk > 128 || dv <= 0 || dv > 128) return ATOM_ERR_ARG;
  if (dtype == ATOM_F32)
    return atom::launch_wkv<float>((float*)y, (const float*)r, (const float*)k, (const float*)v, d, d_dtype,
                                   (const float*)gate, w0, u, norm_w, vec_dtype, state, cu_q, state_slots, S, heads,
                                   dk, dv, eps, write_state, stream);
  if (dtype == ATOM_BF16)
    return atom::launch_wkv<__nv_bfloat16>((__nv_bfloat16*)y, (const __nv_bfloat16*)r, (const __nv_bfloat16*)k,
                                           (const __nv_bfloat16*)v, d, d_dtype, (const __nv_bfloat16*)gate, w0, u,
                                           norm_w, vec_dtype, state, cu_q, state_slots, S, heads, dk, dv, eps,
                                           write_state, stream);
  return ATOM_ERR_ARG;
}
