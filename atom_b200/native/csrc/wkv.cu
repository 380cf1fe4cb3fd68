// Linear recurrence with a decay per key channel and a bonus for the present token, per request and head:
//   o_t[j] = sum_i r_t[i] * (S[i][j] + u[i] * k_t[i] * v_t[j])
//   S[i][j] <- w_t[i] * S[i][j] + k_t[i] * v_t[j],        w_t[i] = exp(-exp(d_t[i] + w0[i]))
// followed by what the mixer does with o before its output product: each head's o divided by its root
// mean square, times a weight per channel, times silu(gate).  The state S [dk, dv] is 32-bit, lives in
// the request's state row between steps, and all arithmetic of the recurrence is 32-bit; r, k, v, d and
// the gate come from matrix products in the activation type.
//
// One block per (request, head); a state column j (the columns do not depend on one another) belongs to
// kWkvSplit neighbouring lanes, each of which keeps a quarter of the column's key channels in registers, so
// a token costs dk / 4 multiply-adds per thread and two shuffles, and the token-to-token chain is short.
// The bonus needs no pass over the state: sum_i r[i] u[i] k[i] v[j] = v[j] * b with one number b per token,
// which is formed while the chunk is staged.  Tokens go through shared memory in chunks: r, k and the decay
// of a chunk are converted (and the two exponentials taken) once, by all threads.  The order of the sums
// does not depend on how a request's tokens are cut into steps or chunks.
#include "common.cuh"

namespace atom {

constexpr int kWkvChunk = 16;
constexpr int kWkvSplit = 4;      // lanes to a state column

template <typename T, int DKP>
__global__ void __launch_bounds__(1024)
wkv_kernel(T* __restrict__ y, const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
           const void* __restrict__ d, int d_dtype, const T* __restrict__ gate, const void* __restrict__ w0,
           const void* __restrict__ u, const void* __restrict__ norm_w, int vec_dtype, float* __restrict__ state,
           const int* __restrict__ cu_q, const int* __restrict__ state_slots, int heads, int dk, int dv,
           float eps, int write_state) {
  atom::pdl_trigger();
  atom::pdl_wait();
  constexpr int DKQ = DKP / kWkvSplit;        // channels per lane (a multiple of 4)
  extern __shared__ __align__(16) float smem[];
  float* r_s = smem;                          // [chunk][DKP]
  float* k_s = r_s + kWkvChunk * DKP;         // [chunk][DKP]
  float* w_s = k_s + kWkvChunk * DKP;         // [chunk][DKP]
  float* u_s = w_s + kWkvChunk * DKP;         // [DKP]
  float* w0_s = u_s + DKP;                    // [DKP]
  float* v_s = w0_s + DKP;                    // [chunk][dv]
  float* o_s = v_s + kWkvChunk * dv;          // [chunk][dv]
  __shared__ float rstd_s[kWkvChunk];
  __shared__ float b_s[kWkvChunk];

  const int s = blockIdx.x, hd = blockIdx.y;
  const int t0 = cu_q[s], t1 = cu_q[s + 1];
  if (t1 <= t0) return;                       // a request without tokens in this step (padding)
  const int j = threadIdx.x / kWkvSplit, part = threadIdx.x % kWkvSplit;
  const int i0 = part * DKQ;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int64_t ldk = (int64_t)heads * dk, ldv = (int64_t)heads * dv;
  float* S_g = state + (((int64_t)state_slots[s] * heads + hd) * dk) * dv;

  for (int i = threadIdx.x; i < DKP; i += blockDim.x) {
    u_s[i] = i < dk ? load_as_float(u, vec_dtype, (int64_t)hd * dk + i) : 0.f;
    w0_s[i] = i < dk ? load_as_float(w0, vec_dtype, (int64_t)hd * dk + i) : 0.f;
  }
  float S[DKQ];
#pragma unroll
  for (int i = 0; i < DKQ; ++i) S[i] = (i0 + i < dk && j < dv) ? S_g[(int64_t)(i0 + i) * dv + j] : 0.f;
  __syncthreads();

  for (int c0 = t0; c0 < t1; c0 += kWkvChunk) {
    const int n = min(kWkvChunk, t1 - c0);
    for (int e = threadIdx.x; e < n * DKP; e += blockDim.x) {
      const int c = e / DKP, i = e - c * DKP;
      float rv = 0.f, kv = 0.f, wv = 1.f;
      if (i < dk) {
        const int64_t off = (int64_t)(c0 + c) * ldk + (int64_t)hd * dk + i;
        rv = to_float(r[off]);
        kv = to_float(k[off]);
        wv = expf(-expf(load_as_float(d, d_dtype, off) + w0_s[i]));
      }
      r_s[e] = rv;
      k_s[e] = kv;
      w_s[e] = wv;
    }
    for (int e = threadIdx.x; e < n * dv; e += blockDim.x) {
      const int c = e / dv, jj = e - c * dv;
      v_s[e] = to_float(v[(int64_t)(c0 + c) * ldv + (int64_t)hd * dv + jj]);
    }
    __syncthreads();
    // the bonus' number of every token: a warp per token, lanes stride over the channels
    for (int c = warp; c < n; c += nwarps) {
      float b = 0.f;
      for (int i = lane; i < DKP; i += 32) b = fmaf(r_s[c * DKP + i] * u_s[i], k_s[c * DKP + i], b);
      b = warp_sum(b);
      if (lane == 0) b_s[c] = b;
    }
    __syncthreads();
    if (j < dv) {
      const unsigned group_mask = 0xFu << (lane & ~3);
      for (int c = 0; c < n; ++c) {
        const float vj = v_s[c * dv + j];
        const float4* rr = reinterpret_cast<const float4*>(r_s + c * DKP + i0);
        const float4* kk = reinterpret_cast<const float4*>(k_s + c * DKP + i0);
        const float4* ww = reinterpret_cast<const float4*>(w_s + c * DKP + i0);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int m = 0; m < DKQ / 4; ++m) {
          const float4 r4 = rr[m], k4 = kk[m], w4 = ww[m];
          a0 = fmaf(r4.x, S[4 * m], a0);
          a1 = fmaf(r4.y, S[4 * m + 1], a1);
          a2 = fmaf(r4.z, S[4 * m + 2], a2);
          a3 = fmaf(r4.w, S[4 * m + 3], a3);
          S[4 * m] = fmaf(w4.x, S[4 * m], k4.x * vj);
          S[4 * m + 1] = fmaf(w4.y, S[4 * m + 1], k4.y * vj);
          S[4 * m + 2] = fmaf(w4.z, S[4 * m + 2], k4.z * vj);
          S[4 * m + 3] = fmaf(w4.w, S[4 * m + 3], k4.w * vj);
        }
        float acc = (a0 + a1) + (a2 + a3);
        acc += __shfl_xor_sync(group_mask, acc, 1);      // (a column's lanes are neighbours in one warp)
        acc += __shfl_xor_sync(group_mask, acc, 2);
        if (part == 0) o_s[c * dv + j] = fmaf(b_s[c], vj, acc);
      }
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
      const float g = to_float(gate[off]);
      const float sg = g / (1.f + expf(-g));
      y[off] = from_float<T>(o_s[e] * rstd_s[c] * load_as_float(norm_w, vec_dtype, (int64_t)hd * dv + jj) * sg);
    }
    __syncthreads();
  }
  if (write_state && j < dv) {
#pragma unroll
    for (int i = 0; i < DKQ; ++i)
      if (i0 + i < dk) S_g[(int64_t)(i0 + i) * dv + j] = S[i];
  }
}

template <typename T>
static int launch_wkv(T* y, const T* r, const T* k, const T* v, const void* d, int d_dtype, const T* gate,
                      const void* w0, const void* u, const void* norm_w, int vec_dtype, float* state,
                      const int* cu_q, const int* state_slots, int S, int heads, int dk, int dv, float eps,
                      int write_state, cudaStream_t stream) {
  const int threads = ((dv * kWkvSplit + 31) / 32) * 32;
  const int dkp = ((dk + 15) / 16) * 16;
  const size_t smem = sizeof(float) * ((size_t)3 * kWkvChunk * dkp + 2 * dkp + (size_t)2 * kWkvChunk * dv);
#define ATOM_WKV_CASE(N)                                                                                         \
  case N:                                                                                                        \
    if (smem > 48 * 1024)                                                                                        \
      cudaFuncSetAttribute(wkv_kernel<T, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);            \
    launch_pdl(wkv_kernel<T, N>, dim3(S, heads), dim3(threads), smem, stream, y, r, k, v, d, d_dtype, gate, w0, \
               u, norm_w, vec_dtype, state, cu_q, state_slots, heads, dk, dv, eps, write_state);                 \
    break;
  switch (dkp) {
    ATOM_WKV_CASE(16)
    ATOM_WKV_CASE(32)
    ATOM_WKV_CASE(48)
    ATOM_WKV_CASE(64)
    ATOM_WKV_CASE(80)
    ATOM_WKV_CASE(96)
    ATOM_WKV_CASE(112)
    ATOM_WKV_CASE(128)
    default:
      return ATOM_ERR_ARG;
  }
#undef ATOM_WKV_CASE
  return check_launch();
}

}  // namespace atom

// y, gate: [T, heads * dv]; r, k, d: [T, heads * dk]; v: [T, heads * dv]; w0, u: [heads * dk]; norm_w: [heads * dv]
// (all three of one type); state: [slots, heads, dk, dv] float32.  d may be float32 beside bf16 activations.
ATOM_EXPORT int atom_wkv(void* y, const void* r, const void* k, const void* v, int dtype, const void* d, int d_dtype,
                         const void* gate, const void* w0, const void* u, const void* norm_w, int vec_dtype,
                         float* state, const int* cu_q, const int* state_slots, int S, int heads, int dk, int dv,
                         float eps, int write_state, cudaStream_t stream) {
  if (S <= 0) return ATOM_OK;
  if (heads <= 0 || heads > 65535 || dk <= 0 || dk > 128 || dv <= 0 || dv > 256) return ATOM_ERR_ARG;
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
