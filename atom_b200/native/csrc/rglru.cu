// A gated linear recurrence per channel with a short causal convolution in front (the recurrent block of
// Griffin, De et al. 2024):
//   v_t = x_t + bx                                   the branch's projection with its bias
//   u_t = bc + sum_k w[c, k] * v_(t - taps + 1 + k)  causal convolution per channel, zeros before the start
//   r_t = sigmoid(gr_t + br),  i_t = sigmoid(gi_t + bi)     gr, gi: block-diagonal products of u (computed outside)
//   a_t = exp(-c * r_t * softplus(lam)),  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t
//   out_t = S_t * gelu_tanh(y_t + by)
// Per request the state row keeps S (32-bit) and the last taps - 1 values of v; both are zero at a request's
// first token.  Gates, decay and state are 32-bit in both precisions.
//
//   causal_conv_kernel   every (token, channel) on its own: values before the step's first token come from
//                        the state row, which this kernel only reads
//   rglru_scan_kernel    a request's tokens of the step in runs, one warp per run and one lane per channel; then S
//                        and the last taps - 1 values of v go back to the state row
#include "common.cuh"
#include <cstdint>

namespace atom {

constexpr int kMaxTaps = 32;

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

// The value of the x branch that enters the convolution, rounded as the state keeps it, so that a value is
// the same whether it is read from this step's rows or, a step later, from the state.
template <typename T>
__device__ __forceinline__ float conv_input(const T* x, int64_t ld, int64_t t, int c, float bias) {
  return to_float(from_float<T>(to_float(x[t * ld + c]) + bias));
}

// x: [T, ld] (the branch's columns start at x itself); u: [T, W]; conv_state: [slots, taps - 1, W], oldest first.
// A thread owns a channel and TS consecutive rows of the step: its taps and the TS + taps - 1 inputs it needs are
// read once.  Tap k of the design is slot k + KT - taps of KT >= taps here, so that every index is known at compile
// time.
template <typename T, int TS, int KT>
__global__ void causal_conv_kernel(T* __restrict__ u, const T* __restrict__ x, int64_t ld,
                                   const void* __restrict__ bx, const void* __restrict__ w,
                                   const void* __restrict__ bc, int w_dtype, const T* __restrict__ conv_state,
                                   const int* __restrict__ seq_of_token, const int* __restrict__ cu_q,
                                   const int* __restrict__ state_slots, int n_rows, int W, int taps) {
  atom::pdl_trigger();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int t_base = blockIdx.x * TS;
  if (c >= W) return;
  const int skip = KT - taps;
  float wt[KT];
#pragma unroll
  for (int k = 0; k < KT; ++k) wt[k] = k >= skip ? load_as_float(w, w_dtype, (int64_t)c * taps + k - skip) : 0.f;
  const float bias = load_as_float(bx, w_dtype, c), cbias = load_as_float(bc, w_dtype, c);
  atom::pdl_wait();
  float xv[TS + KT - 1];
#pragma unroll
  for (int j = 0; j < TS + KT - 1; ++j) {
    const int i = t_base - (KT - 1) + j;
    xv[j] = (j >= skip && i >= 0 && i < n_rows) ? conv_input(x, ld, i, c, bias) : 0.f;
  }
#pragma unroll
  for (int tt = 0; tt < TS; ++tt) {
    const int t = t_base + tt;
    if (t >= n_rows) break;
    const int s = seq_of_token[t];
    if (s < 0) continue;
    const int first = cu_q[s];
    float acc = cbias;
    if (t - (taps - 1) >= first) {
#pragma unroll
      for (int k = 0; k < KT; ++k) acc = fmaf(wt[k], xv[tt + k], acc);
    } else {      // the request's first rows of the step: what came before them is in its state
      const T* st = conv_state + (int64_t)state_slots[s] * (taps - 1) * W;
#pragma unroll
      for (int k = 0; k < KT; ++k) {
        const int i = t - (KT - 1) + k;
        if (k < skip) continue;
        const float v = i >= first ? xv[tt + k] : to_float(st[(int64_t)(taps - 1 + i - first) * W + c]);
        acc = fmaf(wt[k], v, acc);
      }
    }
    u[(int64_t)t * W + c] = from_float<T>(acc);
  }
}

// gates: [T, blocks, 2 * bw] float (r's sums, then i's, per block of bw channels); gate_b: [blocks, 2 * bw];
// y, x: [T, ld] columns of the two branches before bias; out: [T, W].
// A block is cw channels (32, or 16 where long portions would otherwise leave SMs idle) x NW warps; a request's
// tokens of the step are cut into runs, one per group of cw lanes.  The recurrence is linear in S, so a run is
// summed up as S_end = A S_begin + B: every group first finds (A, B) of its run, the pairs of the runs before it give
// its S_begin, and a second walk writes the outputs.  Few tokens (a decoded token above all) are walked once, by the
// first group.
constexpr int kScanOnce = 8;      // up to this many tokens of a request: one walk

template <typename T>
__global__ void __launch_bounds__(1024)
rglru_scan_kernel(T* __restrict__ out, const float* __restrict__ gates, const void* __restrict__ gate_b,
                  const void* __restrict__ lam, const T* __restrict__ u, const T* __restrict__ y,
                  const T* __restrict__ x, int64_t ld, const void* __restrict__ by, const void* __restrict__ bx,
                  int w_dtype, float* __restrict__ state, T* __restrict__ conv_state, const int* __restrict__ cu_q,
                  const int* __restrict__ state_slots, int W, int bw, int taps, float decay_c, int write_state,
                  int cw) {
  atom::pdl_trigger();
  __shared__ float sA[64][33], sB[64][33];
  const int s = blockIdx.x;
  const int lane = threadIdx.x & 31, cl = lane & (cw - 1);
  const int run = (threadIdx.x >> 5) * (32 / cw) + lane / cw, NR = (blockDim.x >> 5) * (32 / cw);
  const int c = blockIdx.y * cw + cl;
  const bool live = c < W;
  const int b = live ? c / bw : 0, cb = live ? c - b * bw : 0;
  float sp = 0.f, br = 0.f, bi = 0.f, byc = 0.f, bxc = 0.f;
  if (live) {       // parameters do not depend on the kernels in front
    sp = decay_c * softplus_f(load_as_float(lam, w_dtype, c));
    br = load_as_float(gate_b, w_dtype, (int64_t)b * 2 * bw + cb);
    bi = load_as_float(gate_b, w_dtype, (int64_t)b * 2 * bw + bw + cb);
    byc = load_as_float(by, w_dtype, c);
    bxc = load_as_float(bx, w_dtype, c);
  }
  atom::pdl_wait();
  const int first = cu_q[s], last = cu_q[s + 1];
  const int n = last - first;
  if (n <= 0) return;
  const bool once = n <= kScanOnce || NR == 1;
  const int per = once ? n : (n + NR - 1) / NR;
  const int t0 = min(last, first + run * per), t1 = min(last, t0 + per);
  const int slot = state_slots[s];
  const int64_t goff = (int64_t)b * 2 * bw + cb;

  // a_t and b_t = sqrt(1 - a_t^2) i_t u_t of token t
  auto step_of = [&](int t, float& a, float& bt) {
    const float* g = gates + (int64_t)t * 2 * W + goff;
    const float r = sigmoid_f(g[0] + br), gi = sigmoid_f(g[bw] + bi);
    const float la = -r * sp;                            // log a
    a = expf(la);
    bt = sqrtf(-expm1f(2.f * la)) * gi * to_float(u[(int64_t)t * W + c]);      // sqrt(1 - a^2) without cancellation near a = 1
  };

  float S = live ? state[(int64_t)slot * W + c] : 0.f;
  if (!once) {
    float A = 1.f, B = 0.f;
    if (live)
      for (int t = t0; t < t1; ++t) {
        float a, bt;
        step_of(t, a, bt);
        A *= a;
        B = fmaf(a, B, bt);
      }
    sA[run][cl] = A;
    sB[run][cl] = B;
    __syncthreads();
    for (int k = 0; k < run; ++k) S = fmaf(sA[k][cl], S, sB[k][cl]);
  }
  if (!live) return;
  for (int t = t0; t < t1; ++t) {
    float a, bt;
    step_of(t, a, bt);
    S = fmaf(a, S, bt);
    const float yv = gelu_tanh_f(to_float(y[(int64_t)t * ld + c]) + byc);
    out[(int64_t)t * W + c] = from_float<T>(S * yv);
  }
  if (!write_state || t1 != last || t0 >= t1) return;       // the warp with the request's last token carries on
  state[(int64_t)slot * W + c] = S;
  // the last taps - 1 convolution inputs: this step's where it has them, else the older ones moved up
  T* st = conv_state + (int64_t)slot * (taps - 1) * W;
  const int keep = taps - 1;
  T old[kMaxTaps];
  for (int k = 0; k < keep; ++k) old[k] = st[(int64_t)k * W + c];
  for (int k = 0; k < keep; ++k) {
    const int i = n - keep + k;       // index into this step's tokens of the request
    st[(int64_t)k * W + c] = i >= 0 ? from_float<T>(to_float(x[(int64_t)(first + i) * ld + c]) + bxc) : old[k + n];
  }
}

// x[t, :] *= sigmoid(g[t, :]) elementwise, x [T, n] dense, g rows ld apart; 32-bit arithmetic.
template <typename T>
__global__ void sigmoid_mul_kernel(T* __restrict__ x, const T* __restrict__ g, int64_t ld, int64_t total, int n) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int64_t t = idx / n;
    const int i = (int)(idx - t * n);
    x[idx] = from_float<T>(to_float(x[idx]) * sigmoid_f(to_float(g[t * ld + i])));
  }
}

// out[t, i] = gelu_tanh(gu[t, i]) * gu[t, I + i], gu [T, 2 I].
template <typename T>
__global__ void gelu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, int64_t n, int I) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += stride) {
    const int64_t t = idx / I;
    const int i = (int)(idx - t * I);
    out[idx] = from_float<T>(gelu_tanh_f(to_float(gu[t * 2 * I + i])) * to_float(gu[t * 2 * I + I + i]));
  }
}

// The two kernels above for bfloat16 rows of a multiple of 8 numbers at 16-byte-aligned places: 16 bytes per load.
__global__ void sigmoid_mul_bf16_vec_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g, int64_t ld,
                                            int64_t nvec, int n8) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nvec; idx += stride) {
    const int64_t t = idx / n8;
    const int i = (int)(idx - t * n8);
    uint4 x4 = *reinterpret_cast<const uint4*>(x + idx * 8);
    const uint4 g4 = *reinterpret_cast<const uint4*>(g + t * ld + (int64_t)i * 8);
    __nv_bfloat162* xh = reinterpret_cast<__nv_bfloat162*>(&x4);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(xh[e]), b = __bfloat1622float2(gh[e]);
      xh[e] = __floats2bfloat162_rn(a.x * sigmoid_f(b.x), a.y * sigmoid_f(b.y));
    }
    *reinterpret_cast<uint4*>(x + idx * 8) = x4;
  }
}

__global__ void gelu_mul_bf16_vec_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gu,
                                         int64_t nvec, int I8) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nvec; idx += stride) {
    const int64_t t = idx / I8;
    const int i = (int)(idx - t * I8);
    const uint4 g4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + i) * 8);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gu + (t * 2 * I8 + I8 + i) * 8);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(gh[e]), b = __bfloat1622float2(uh[e]);
      oh[e] = __floats2bfloat162_rn(gelu_tanh_f(a.x) * b.x, gelu_tanh_f(a.y) * b.y);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = o4;
  }
}

}  // namespace atom

ATOM_EXPORT int atom_causal_conv(void* u, const void* x, int dtype, int64_t ld, const void* bx, const void* w,
                                 const void* bc, int w_dtype, const void* conv_state, const int* seq_of_token,
                                 const int* cu_q, const int* state_slots, int T, int W, int taps, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (W <= 0 || taps < 1 || taps > atom::kMaxTaps || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16)) return ATOM_ERR_ARG;
  const int threads = 128;
  const int gy = (W + threads - 1) / threads;
  if (gy > 65535) return ATOM_ERR_ARG;
  // strips of 8 rows per thread in long steps, a row per thread in short ones (by the step's size alone); tap slots
  // in steps of 8, 16, 32
#define ATOM_CONV(TYPE, TS, KT)                                                                                         \
  atom::launch_pdl(atom::causal_conv_kernel<TYPE, TS, KT>, dim3((T + TS - 1) / TS, gy), dim3(threads), 0, stream,       \
                   (TYPE*)u, (const TYPE*)x, ld, bx, w, bc, w_dtype, (const TYPE*)conv_state, seq_of_token, cu_q,       \
                   state_slots, T, W, taps)
#define ATOM_CONV_T(TYPE)                                                    \
  do {                                                                       \
    if (taps <= 8) {                                                         \
      if (T >= 256) ATOM_CONV(TYPE, 8, 8); else ATOM_CONV(TYPE, 1, 8);       \
    } else if (taps <= 16) {                                                 \
      if (T >= 256) ATOM_CONV(TYPE, 8, 16); else ATOM_CONV(TYPE, 1, 16);     \
    } else {                                                                 \
      if (T >= 256) ATOM_CONV(TYPE, 4, 32); else ATOM_CONV(TYPE, 1, 32);     \
    }                                                                        \
  } while (0)
  if (dtype == ATOM_F32) ATOM_CONV_T(float);
  else if (dtype == ATOM_BF16) ATOM_CONV_T(__nv_bfloat16);
  else return ATOM_ERR_ARG;
#undef ATOM_CONV_T
#undef ATOM_CONV
  return atom::check_launch();
}

ATOM_EXPORT int atom_rglru_scan(void* out, const float* gates, const void* gate_b, const void* lam, const void* u,
                                const void* y, const void* x, int dtype, int64_t ld, const void* by, const void* bx,
                                int w_dtype, float* state, void* conv_state, const int* cu_q, const int* state_slots,
                                int num_seqs, int T, int W, int bw, int taps, float decay_c, int write_state,
                                cudaStream_t stream) {
  if (num_seqs <= 0 || T <= 0) return ATOM_OK;
  if (W <= 0 || bw <= 0 || W % bw || taps < 1 || taps > atom::kMaxTaps || (w_dtype != ATOM_F32 && w_dtype != ATOM_BF16))
    return ATOM_ERR_ARG;
  // warps along the tokens: by the step's size alone, so that a captured step replays the same launch
  const int threads = 32 * (T >= 512 ? 32 : (T >= 32 ? 8 : 1));
  const int cw = (T >= 512 && num_seqs * ((W + 31) / 32) < 148) ? 16 : 32;
  const dim3 grid(num_seqs, (W + cw - 1) / cw);
  if (grid.y > 65535) return ATOM_ERR_ARG;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::rglru_scan_kernel<float>, grid, dim3(threads), 0, stream, (float*)out, gates, gate_b, lam,
                     (const float*)u, (const float*)y, (const float*)x, ld, by, bx, w_dtype, state, (float*)conv_state,
                     cu_q, state_slots, W, bw, taps, decay_c, write_state, cw);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::rglru_scan_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)out, gates,
                     gate_b, lam, (const __nv_bfloat16*)u, (const __nv_bfloat16*)y, (const __nv_bfloat16*)x, ld, by, bx,
                     w_dtype, state, (__nv_bfloat16*)conv_state, cu_q, state_slots, W, bw, taps, decay_c, write_state,
                     cw);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

ATOM_EXPORT int atom_sigmoid_mul(void* x, const void* g, int dtype, int64_t ld, int T, int n, cudaStream_t stream) {
  if (T <= 0 || n <= 0) return ATOM_OK;
  const int64_t total = (int64_t)T * n;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == ATOM_BF16 && n % 8 == 0 && ld % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)g % 16 == 0) {
    const int64_t nvec = total / 8;
    int64_t vb = (nvec + 255) / 256;
    if (vb > 148 * 32) vb = 148 * 32;
    atom::launch_pdl(atom::sigmoid_mul_bf16_vec_kernel, dim3((int)vb), dim3(256), 0, stream, (__nv_bfloat16*)x,
                     (const __nv_bfloat16*)g, ld, nvec, n / 8);
    return atom::check_launch();
  }
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::sigmoid_mul_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (float*)x, (const float*)g, ld, total, n);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::sigmoid_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, (__nv_bfloat16*)x, (const __nv_bfloat16*)g, ld, total, n);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

ATOM_EXPORT int atom_gelu_mul(void* out, const void* gu, int dtype, int T, int I, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (I <= 0) return ATOM_ERR_ARG;
  const int64_t n = (int64_t)T * I;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == ATOM_BF16 && I % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gu % 16 == 0) {
    const int64_t nvec = n / 8;
    int64_t vb = (nvec + 255) / 256;
    if (vb > 148 * 32) vb = 148 * 32;
    atom::launch_pdl(atom::gelu_mul_bf16_vec_kernel, dim3((int)vb), dim3(256), 0, stream, (__nv_bfloat16*)out,
                     (const __nv_bfloat16*)gu, nvec, I / 8);
    return atom::check_launch();
  }
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::gelu_mul_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (float*)out, (const float*)gu, n, I);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::gelu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, (__nv_bfloat16*)out, (const __nv_bfloat16*)gu, n, I);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}
