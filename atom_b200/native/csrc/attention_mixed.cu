// Causal attention over the paged cache whose heads see one another's scores:
//   s_g[j]  = scale * temp(p) * (q_g . k_j) + rel[bucket(p - j)][g]        per query head g, key j <= p
//   s'_h[j] = sum_g mix[h][g] * s_g[j]                                       scores mixed across heads
//   w_h[j]  = exp(s'_h[j]) / (exp(sink_h) + sum_j' exp(s'_h[j']))            softmax with a sink per head
//   o_h     = sum_j w_h[j] * v_j                                             (values of the head's kv head)
// temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1) scales the query of position p; bucket() maps a
// distance to a row of the bias table: the distance itself below `half`, above it the rows follow
// thresholds that the host computed (ascending distances at which the next row begins).  Every one of
// these is optional (null pointer / zero count).  Scores, weights and sums are 32-bit; queries, keys
// and values have the activation type.  Key size and value size may differ.
//
// This is the plain kernel for any sizes: one block per query token takes all heads (the mixing needs
// all heads' scores of a key at once) and walks the token's keys in chunks with a running maximum and
// sum per head, which start at the sink's value and at one.  With few tokens in the step (decoding) the keys
// of a token are shared out among `nsplit` blocks, each of which leaves its maximum, sum and unnormalised
// output per head in a scratch array; a second kernel puts them together.
#include "common.cuh"

namespace atom {

constexpr int kMixThreads = 256;
constexpr int kMixChunk = 64;
constexpr int kMixMaxAcc = 32;      // outputs per thread: heads * value size <= 32 * 256

// Row of the bias table for distance n.
__device__ __forceinline__ int distance_bucket(int n, int half, const int* __restrict__ thr, int n_thr) {
  if (n < half) return n;
  int b = 0;
  for (int k = 0; k < n_thr; ++k) b += (thr[k] <= n) ? 1 : 0;     // thresholds ascend
  return half + b;
}

__device__ __forceinline__ float query_temperature(int p, float coef, int every) {
  if (every <= 0) return 1.f;
  return 1.f + coef * logf((float)((p + 1) / every) + 1.f);
}

// Writes a step's keys and values to their pages; each value head is first divided by its root mean
// square (no weight) when vnorm is set.  One block per token, one warp per kv head at a time.
template <typename T>
__global__ void kv_write_kernel(const T* __restrict__ qkv, int64_t ld, int k_off, int v_off, int nkv, int dk, int dv,
                                int vnorm, float eps, const int* __restrict__ positions,
                                const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                int max_pages, int page_size, T* __restrict__ k_pages, T* __restrict__ v_pages,
                                int64_t num_pages, int* __restrict__ status) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  if (s < 0) return;
  const int p = positions[t];
  const int lp = p / page_size;
  const int page = lp < max_pages ? block_table[(int64_t)s * max_pages + lp] : -1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    return;
  }
  const T* row = qkv + (int64_t)t * ld;
  for (int g = warp; g < nkv; g += nwarps) {
    const int64_t slot = ((int64_t)page * nkv + g) * page_size + (p % page_size);
    const T* ks = row + k_off + g * dk;
    T* kd = k_pages + slot * dk;
    for (int i = lane; i < dk; i += 32) kd[i] = ks[i];
    const T* vs = row + v_off + g * dv;
    T* vd = v_pages + slot * dv;
    float rstd = 1.f;
    if (vnorm) {
      float ss = 0.f;
      for (int i = lane; i < dv; i += 32) {
        const float x = to_float(vs[i]);
        ss = fmaf(x, x, ss);
      }
      ss = warp_sum(ss);
      rstd = rsqrtf(ss / (float)dv + eps);
    }
    for (int i = lane; i < dv; i += 32) vd[i] = vnorm ? from_float<T>(to_float(vs[i]) * rstd) : vs[i];
  }
}

template <typename T>
__global__ void __launch_bounds__(kMixThreads)
attention_mixed_kernel(T* __restrict__ out, const T* __restrict__ q, int64_t q_stride, const T* __restrict__ k_pages,
                       const T* __restrict__ v_pages, const int* __restrict__ block_table, int max_pages,
                       int page_size, const int* __restrict__ positions, const int* __restrict__ seq_of_token, int nh,
                       int nkv, int dk, int dv, float scale, int window, const float* __restrict__ rel, int half,
                       const int* __restrict__ thr, int n_thr, const float* __restrict__ mix,
                       const float* __restrict__ sink, float temp_coef, int temp_every, int nsplit,
                       float* __restrict__ part) {
  atom::pdl_trigger();
  atom::pdl_wait();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* q_s = (float*)smem_raw;                 // [nh][dk]
  float* s_s = q_s + nh * dk;                    // [nh][chunk]  raw scores with bias
  float* p_s = s_s + nh * kMixChunk;             // [nh][chunk]  mixed scores, then weights
  float* mix_s = p_s + nh * kMixChunk;           // [nh][nh] (if mixing)
  float* m_s = mix_s + (mix ? nh * nh : 0);      // [nh] running maximum
  float* l_s = m_s + nh;                         // [nh] running sum
  float* c_s = l_s + nh;                         // [nh] correction of this chunk
  int* page_s = (int*)(c_s + nh);                // [chunk]
  int* bkt_s = page_s + kMixChunk;               // [chunk]
  int* thr_s = bkt_s + kMixChunk;                // [n_thr]

  const int t = blockIdx.x;
  if (seq_of_token[t] < 0) return;
  const int p = positions[t];
  const int* bt = block_table + (int64_t)seq_of_token[t] * max_pages;
  const int group = nh / nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int nwarps = kMixThreads / 32;

  const float qf = scale * query_temperature(p, temp_coef, temp_every);
  for (int i = threadIdx.x; i < nh * dk; i += kMixThreads)
    q_s[i] = to_float(q[(int64_t)t * q_stride + i]) * qf;
  if (mix)
    for (int i = threadIdx.x; i < nh * nh; i += kMixThreads) mix_s[i] = mix[i];
  for (int i = threadIdx.x; i < n_thr; i += kMixThreads) thr_s[i] = thr[i];
  const int split = blockIdx.y;
  for (int h = threadIdx.x; h < nh; h += kMixThreads) {      // the sink counts once: in the first share
    m_s[h] = (sink && split == 0) ? sink[h] : -INFINITY;
    l_s[h] = (sink && split == 0) ? 1.f : 0.f;
  }
  float acc[kMixMaxAcc];
#pragma unroll
  for (int a = 0; a < kMixMaxAcc; ++a) acc[a] = 0.f;
  const int n_out = nh * dv;
  int lo = 0;
  if (window > 0 && p - window + 1 > 0) lo = p - window + 1;
  int hi = p + 1;
  if (nsplit > 1) {      // this block's share of the keys: whole chunks, the first shares full
    const int per = ((p + 1 - lo + nsplit - 1) / nsplit + kMixChunk - 1) / kMixChunk * kMixChunk;
    lo += split * per;
    hi = min(hi, lo + per);
  }
  __syncthreads();

  for (int c0 = lo; c0 < hi; c0 += kMixChunk) {
    const int n = min(kMixChunk, hi - c0);
    for (int jj = threadIdx.x; jj < n; jj += kMixThreads) {
      const int j = c0 + jj;
      page_s[jj] = bt[j / page_size] * page_size + (j % page_size);     // (page, place) folded; kv head added below
      bkt_s[jj] = rel ? distance_bucket(p - j, half, thr_s, n_thr) : 0;
    }
    __syncthreads();
    // raw scores: a warp takes one (kv head, key) at a time and all query heads of the group
    for (int e = warp; e < nkv * n; e += nwarps) {
      const int g = e / n, jj = e - g * n;
      const int pg = page_s[jj] / page_size, pl = page_s[jj] - pg * page_size;
      const T* kr = k_pages + (((int64_t)pg * nkv + g) * page_size + pl) * dk;
      for (int hq = 0; hq < group; ++hq) {
        const int h = g * group + hq;
        const float* qh = q_s + h * dk;
        float sacc = 0.f;
        for (int i = lane; i < dk; i += 32) sacc = fmaf(qh[i], to_float(kr[i]), sacc);
        sacc = warp_sum(sacc);
        if (lane == 0) s_s[h * kMixChunk + jj] = sacc + (rel ? rel[bkt_s[jj] * nh + h] : 0.f);
      }
    }
    __syncthreads();
    // mixing across heads
    for (int e = threadIdx.x; e < nh * n; e += kMixThreads) {
      const int h = e / n, jj = e - h * n;
      float v;
      if (mix) {
        v = 0.f;
        for (int g = 0; g < nh; ++g) v = fmaf(mix_s[h * nh + g], s_s[g * kMixChunk + jj], v);
      } else {
        v = s_s[h * kMixChunk + jj];
      }
      p_s[h * kMixChunk + jj] = v;
    }
    __syncthreads();
    // running softmax: a warp per head
    for (int h = warp; h < nh; h += nwarps) {
      float cm = -INFINITY;
      for (int jj = lane; jj < n; jj += 32) cm = fmaxf(cm, p_s[h * kMixChunk + jj]);
      cm = warp_max(cm);
      const float m_old = m_s[h];
      const float m_new = fmaxf(m_old, cm);
      float ls = 0.f;
      for (int jj = lane; jj < n; jj += 32) {
        const float e = expf(p_s[h * kMixChunk + jj] - m_new);
        p_s[h * kMixChunk + jj] = e;
        ls += e;
      }
      ls = warp_sum(ls);
      if (lane == 0) {
        const float corr = expf(m_old - m_new);      // 0 on the first chunk without a sink
        c_s[h] = corr;
        l_s[h] = l_s[h] * corr + ls;
        m_s[h] = m_new;
      }
    }
    __syncthreads();
    // weights times values: thread owns outputs (h, d) = idx, idx + threads, ...
#pragma unroll
    for (int a = 0; a < kMixMaxAcc; ++a) {
      const int idx = threadIdx.x + a * kMixThreads;
      if (idx < n_out) {
        const int h = idx / dv, d = idx - h * dv;
        const int g = h / group;
        float sacc = acc[a] * c_s[h];
        const float* ph = p_s + h * kMixChunk;
        for (int jj = 0; jj < n; ++jj) {
          const int pg = page_s[jj] / page_size, pl = page_s[jj] - pg * page_size;
          sacc = fmaf(ph[jj], to_float(v_pages[(((int64_t)pg * nkv + g) * page_size + pl) * dv + d]), sacc);
        }
        acc[a] = sacc;
      }
    }
    __syncthreads();
  }
  if (nsplit > 1) {
    float* pt = part + ((int64_t)t * nsplit + split) * (n_out + 2 * nh);
    for (int h = threadIdx.x; h < nh; h += kMixThreads) {
      pt[h] = m_s[h];
      pt[nh + h] = l_s[h];
    }
#pragma unroll
    for (int a = 0; a < kMixMaxAcc; ++a) {
      const int idx = threadIdx.x + a * kMixThreads;
      if (idx < n_out) pt[2 * nh + idx] = acc[a];
    }
    return;
  }
#pragma unroll
  for (int a = 0; a < kMixMaxAcc; ++a) {
    const int idx = threadIdx.x + a * kMixThreads;
    if (idx < n_out) {
      const int h = idx / dv;
      out[(int64_t)t * n_out + idx] = from_float<T>(acc[a] / l_s[h]);
    }
  }
}

// Puts the shares of a token's keys together: per head the largest maximum M, the sums and outputs
// rescaled by exp(m - M).  A share without keys has m = -inf and weighs nothing; the first share is
// never empty.
template <typename T>
__global__ void attention_mixed_merge_kernel(T* __restrict__ out, const float* __restrict__ part,
                                             const int* __restrict__ seq_of_token, int nh, int dv, int nsplit) {
  atom::pdl_trigger();
  atom::pdl_wait();
  const int t = blockIdx.x;
  if (seq_of_token[t] < 0) return;
  const int n_out = nh * dv, stride = n_out + 2 * nh;
  const float* pt = part + (int64_t)t * nsplit * stride;
  for (int idx = threadIdx.x; idx < n_out; idx += blockDim.x) {
    const int h = idx / dv;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, pt[(int64_t)s * stride + h]);
    float L = 0.f, o = 0.f;
    for (int s = 0; s < nsplit; ++s) {
      const float m = pt[(int64_t)s * stride + h];
      const float w = (m == -INFINITY) ? 0.f : expf(m - M);
      L = fmaf(pt[(int64_t)s * stride + nh + h], w, L);
      o = fmaf(pt[(int64_t)s * stride + 2 * nh + idx], w, o);
    }
    out[(int64_t)t * n_out + idx] = from_float<T>(o / L);
  }
}

}  // namespace atom

ATOM_EXPORT int atom_kv_write(const void* qkv, int dtype, int64_t ld, int k_off, int v_off, int T, int nkv, int dk,
                              int dv, int vnorm, float eps, const int* positions, const int* seq_of_token,
                              const int* block_table, int max_pages, int page_size, void* k_pages, void* v_pages,
                              int64_t num_pages, int* status, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (nkv <= 0 || dk <= 0 || dv <= 0 || page_size <= 0) return ATOM_ERR_ARG;
  const int threads = nkv >= 8 ? 256 : (nkv >= 4 ? 128 : 64);
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::kv_write_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)qkv, ld, k_off,
                     v_off, nkv, dk, dv, vnorm, eps, positions, seq_of_token, block_table, max_pages, page_size,
                     (float*)k_pages, (float*)v_pages, num_pages, status);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::kv_write_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream,
                     (const __nv_bfloat16*)qkv, ld, k_off, v_off, nkv, dk, dv, vnorm, eps, positions, seq_of_token,
                     block_table, max_pages, page_size, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, num_pages,
                     status);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

// Puts together the shares that another kernel (attention_mixed_tc.cu) left in `part`.
ATOM_EXPORT int atom_attention_mixed_merge(void* out, int dtype, const float* part, const int* seq_of_token, int T,
                                           int nh, int dv, int nsplit, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (nsplit < 1 || part == nullptr) return ATOM_ERR_ARG;
  if (dtype == ATOM_F32)
    atom::launch_pdl(atom::attention_mixed_merge_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)out, part,
                     seq_of_token, nh, dv, nsplit);
  else if (dtype == ATOM_BF16)
    atom::launch_pdl(atom::attention_mixed_merge_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream,
                     (__nv_bfloat16*)out, part, seq_of_token, nh, dv, nsplit);
  else
    return ATOM_ERR_ARG;
  return atom::check_launch();
}

// out: [T, nh * dv]; q: row t at q + t * q_stride, heads packed [nh, dk]; k_pages [pages, nkv, page, dk];
// v_pages [pages, nkv, page, dv].  rel: [half + n_thr + 1, nh] float32 or null; thr: n_thr ascending distances;
// mix: [nh, nh] float32 or null; sink: [nh] float32 or null; temp_every <= 0: no query temperature.
// nsplit > 1: every token's keys are shared out among nsplit blocks; part: T * nsplit * nh * (dv + 2) floats.
ATOM_EXPORT int atom_attention_mixed(void* out, const void* q, int64_t q_stride, int dtype, const void* k_pages,
                                     const void* v_pages, const int* block_table, int max_pages, int page_size,
                                     const int* positions, const int* seq_of_token, int T, int nh, int nkv, int dk,
                                     int dv, float scale, int window, const float* rel, int half, const int* thr,
                                     int n_thr, const float* mix, const float* sink, float temp_coef, int temp_every,
                                     int nsplit, float* part, cudaStream_t stream) {
  if (T <= 0) return ATOM_OK;
  if (nsplit < 1 || nsplit > 65535 || (nsplit > 1 && part == nullptr)) return ATOM_ERR_ARG;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || dk <= 0 || dv <= 0 || page_size <= 0 ||
      nh * dv > atom::kMixMaxAcc * atom::kMixThreads)
    return ATOM_ERR_ARG;
  const size_t smem = sizeof(float) * ((size_t)nh * dk + 2 * (size_t)nh * atom::kMixChunk + (mix ? nh * nh : 0) +
                                       3 * (size_t)nh) +
                      sizeof(int) * (2 * atom::kMixChunk + (size_t)n_thr);
  if (smem > 200 * 1024) return ATOM_ERR_ARG;
#define ATOM_MIX_LAUNCH(TT)                                                                                        \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      cudaFuncSetAttribute(atom::attention_mixed_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                           (int)smem);                                                                             \
    atom::launch_pdl(atom::attention_mixed_kernel<TT>, dim3(T, nsplit), dim3(atom::kMixThreads), smem, stream,    \
                     (TT*)out, (const TT*)q, q_stride, (const TT*)k_pages, (const TT*)v_pages, block_table,       \
                     max_pages, page_size, positions, seq_of_token, nh, nkv, dk, dv, scale, window, rel, half,    \
                     thr, n_thr, mix, sink, temp_coef, temp_every, nsplit, part);                                  \
    if (nsplit > 1)                                                                                                \
      atom::launch_pdl(atom::attention_mixed_merge_kernel<TT>, dim3(T), dim3(256), 0, stream, (TT*)out,            \
                       (const float*)part, seq_of_token, nh, dv, nsplit);                                          \
  } while (0)
  if (dtype == ATOM_F32)
    ATOM_MIX_LAUNCH(float);
  else if (dtype == ATOM_BF16)
    ATOM_MIX_LAUNCH(__nv_bfloat16);
  else
    return ATOM_ERR_ARG;
#undef ATOM_MIX_LAUNCH
  return atom::check_launch();
}
