// Layer norm (weight, no bias) fused with the residual sum; token shift; token embedding with
// sinusoidal positions and layer norm in one kernel.
//
//   layer norm   r += d;  y = (r - mean(r)) / sqrt(mean((r - mean(r))^2) + eps) * w     float32 throughout
//   token shift  s_t = h_t + (h_{t-1} - h_t) * mu, h_{-1} = what the request's state slot holds (zeros at first);
//                the slot then takes the last h of the step
//   embedding    x = E[id] + P(pos),  P[2i] = sin(pos * base^(-2i/H)), P[2i+1] = cos(same);  out = layer norm(x)
//
// A row is summed by a block whose size depends on the row length alone, so a row's result does not depend
// on what else is in the batch.  The mean is taken first and the deviations are squared afterwards (two
// passes over the row in shared memory), which keeps the variance exact for rows with a large mean.
#include "common.cuh"
#include <initializer_list>

namespace {

__device__ __forceinline__ float inv_sqrt_exact(float v) { return 1.0f / sqrtf(v); }

int norm_threads(int hidden) {
  int threads = 64;
  while (threads < 1024 && threads * 4 < hidden) threads <<= 1;
  return threads;
}

// One block per output row.  Source row = rows ? rows[blockIdx.x] : blockIdx.x.  out (engine type) and out32
// (float32) may each be null; in gather mode the residual is left as it is.
template <typename TD, typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials,
                                     long long partial_stride, const float* __restrict__ weight, float eps,
                                     TO* __restrict__ out, float* __restrict__ out32, const int* __restrict__ rows,
                                     int hidden, int write_residual) {
  pdl_enter();
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  const int src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r = residual + (size_t)src * hidden;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = r[i];
    if (delta) {
      const TD* d = delta + (size_t)src * hidden + i;
      for (int p = 0; p < n_partials; ++p) v += Num<TD>::to_f(d[(size_t)p * partial_stride]);
    }
    row_buf[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, red) / (float)hidden;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = row_buf[i] - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = inv_sqrt_exact(block_sum(sq, red) / (float)hidden + eps);
  TO* o = out ? out + (size_t)blockIdx.x * hidden : nullptr;
  float* o32 = out32 ? out32 + (size_t)blockIdx.x * hidden : nullptr;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = row_buf[i];
    if (write_residual) r[i] = v;
    const float y = (v - mean) * rstd * weight[i];
    if (o) o[i] = Num<TO>::from_f(y);
    if (o32) o32[i] = y;
  }
}

// The same for a step of single tokens, with the token shift and the state update in the same kernel: row t
// belongs to entry t, the token before it is what the slot holds.
template <typename TD, typename TO>
__global__ void add_layernorm_shift1_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials,
                                            long long partial_stride, const float* __restrict__ weight, float eps,
                                            const float* __restrict__ mu, float* __restrict__ state,
                                            const int* __restrict__ entry_slot, TO* __restrict__ out,
                                            TO* __restrict__ shifted, int hidden) {
  pdl_enter();
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  const int row = blockIdx.x;
  float* r = residual + (size_t)row * hidden;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = r[i];
    if (delta) {
      const TD* d = delta + (size_t)row * hidden + i;
      for (int p = 0; p < n_partials; ++p) v += Num<TD>::to_f(d[(size_t)p * partial_stride]);
    }
    row_buf[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, red) / (float)hidden;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = row_buf[i] - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = inv_sqrt_exact(block_sum(sq, red) / (float)hidden + eps);
  float* st = state + (size_t)entry_slot[row] * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = row_buf[i];
    r[i] = v;
    const float y = (v - mean) * rstd * weight[i];
    const float before = st[i];
    st[i] = y;
    out[(size_t)row * hidden + i] = Num<TO>::from_f(y);
    shifted[(size_t)row * hidden + i] = Num<TO>::from_f(y + (before - y) * mu[i]);
  }
}

// The two kernels above for rows whose length is a multiple of 4 (up to 8,192) on 16-byte boundaries: 256 threads a
// row, thread t holds the groups of four elements t, t + 256, ... in registers between the sums and the output, so
// a row is read once and written once.  SHIFT: the single-token kernel (row = entry; mu, state and shifted are used).
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const bf16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 u;
  u.x = *reinterpret_cast<unsigned*>(&a);
  u.y = *reinterpret_cast<unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

template <typename TD, typename TO, int J, bool SHIFT>
__global__ void __launch_bounds__(256)
add_layernorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta, int n_partials, long long partial_stride,
                         const float* __restrict__ weight, float eps, TO* __restrict__ out, float* __restrict__ out32,
                         const int* __restrict__ rows, int hidden, int write_residual, const float* __restrict__ mu,
                         float* __restrict__ state, const int* __restrict__ entry_slot, TO* __restrict__ shifted) {
  pdl_enter();
  __shared__ float red[32];
  const int groups = hidden >> 2;
  const int src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* r = residual + (size_t)src * hidden;
  float4 v[J];
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int gi = threadIdx.x + j * 256;
    if (gi < groups) {
      float4 x = ld4(r + 4 * gi);
      if (delta) {
        const TD* d = delta + (size_t)src * hidden + 4 * gi;
        for (int p = 0; p < n_partials; ++p) {
          const float4 y = ld4(d + (size_t)p * partial_stride);
          x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
        }
      }
      v[j] = x;
      sum += (x.x + x.y) + (x.z + x.w);
    }
  }
  const float mean = block_sum(sum, red) / (float)hidden;
  float sq = 0.0f;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    if (threadIdx.x + j * 256 < groups) {
      const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
      sq = fmaf(d, d, fmaf(c, c, fmaf(b, b, fmaf(a, a, sq))));
    }
  }
  const float rstd = inv_sqrt_exact(block_sum(sq, red) / (float)hidden + eps);
  float* st = SHIFT ? state + (size_t)entry_slot[blockIdx.x] * hidden : nullptr;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int gi = threadIdx.x + j * 256;
    if (gi < groups) {
      const float4 w = ld4(weight + 4 * gi);
      if (write_residual) st4(r + 4 * gi, v[j]);
      const float4 y = make_float4((v[j].x - mean) * rstd * w.x, (v[j].y - mean) * rstd * w.y, (v[j].z - mean) * rstd * w.z,
                                   (v[j].w - mean) * rstd * w.w);
      const size_t at = (size_t)blockIdx.x * hidden + 4 * gi;
      if (out) st4(out + at, y);
      if (out32) st4(out32 + at, y);
      if (SHIFT) {
        const float4 b = ld4(st + 4 * gi), m = ld4(mu + 4 * gi);
        st4(st + 4 * gi, y);
        st4(shifted + at, make_float4(y.x + (b.x - y.x) * m.x, y.y + (b.y - y.y) * m.y, y.z + (b.z - y.z) * m.z,
                                      y.w + (b.w - y.w) * m.w));
      }
    }
  }
}

template <typename TD, typename TO, bool SHIFT>
int launch_layernorm_vec(float* residual, const void* delta, int n_partials, long long partial_stride, const float* weight,
                         float eps, void* out, float* out32, const int* rows, int n_rows, int hidden, int write_residual,
                         const float* mu, float* state, const int* entry_slot, void* shifted, cudaStream_t stream) {
  int rc = IFX_ERR_UNSUPPORTED;
#define IFX_LNV(J) case J: rc = launch_pdl(add_layernorm_vec_kernel<TD, TO, J, SHIFT>, dim3(n_rows), dim3(256), 0, stream, residual, \
    (const TD*)delta, n_partials, partial_stride, weight, eps, (TO*)out, out32, rows, hidden, write_residual, mu, state,       \
    entry_slot, (TO*)shifted); break;
  switch ((hidden / 4 + 255) / 256) {
    IFX_LNV(1) IFX_LNV(2) IFX_LNV(3) IFX_LNV(4) IFX_LNV(5) IFX_LNV(6) IFX_LNV(7) IFX_LNV(8)
    default: return IFX_ERR_UNSUPPORTED;
  }
#undef IFX_LNV
  return rc ? rc : IFX_LAUNCH_CHECK();
}

// Whether the vector kernels take these operands (a property of the row length and the addresses, never of the batch).
bool vec_ok(int hidden, long long partial_stride, std::initializer_list<const void*> ptrs) {
  if (hidden % 4 || hidden > 4 * 8 * 256 || (partial_stride & 3)) return false;
  for (const void* p : ptrs)
    if ((uintptr_t)p & 15) return false;
  return true;
}

// One block per row.  h32: the normed rows in float32.  The block of an entry's first row reads what the slot
// holds and, element by element after that, puts the entry's last row there; no other block touches the slot.
template <typename TO>
__global__ void token_shift_kernel(const float* __restrict__ h32, const float* __restrict__ mu, float* __restrict__ state,
                                   const int* __restrict__ row_entry, const int* __restrict__ entry_q_start,
                                   const int* __restrict__ entry_q_len, const int* __restrict__ entry_slot,
                                   TO* __restrict__ out, int hidden) {
  pdl_enter();
  const int row = blockIdx.x;
  const int e = row_entry[row];
  const int q0 = entry_q_start[e];
  const bool first = row == q0;
  const float* h = h32 + (size_t)row * hidden;
  float* st = state + (size_t)entry_slot[e] * hidden;
  const float* before = first ? st : h - hidden;
  const float* last = h32 + (size_t)(q0 + entry_q_len[e] - 1) * hidden;
  TO* o = out + (size_t)row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float b = before[i], v = h[i];
    o[i] = Num<TO>::from_f(v + (b - v) * mu[i]);
    if (first) st[i] = last[i];
  }
}

// One block per token: gather, add the position vector (angles in float64, rounded once), layer norm.
template <typename T>
__global__ void embed_sinusoid_layernorm_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                                const int* __restrict__ positions, const float* __restrict__ weight,
                                                float eps, double log_base, float* __restrict__ out, int hidden, int vocab) {
  pdl_enter();
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;       // never read outside the table
  const T* row = table + (size_t)(ok ? id : 0) * hidden;
  const double pos = (double)positions[t];
  float sum = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const double angle = pos * exp(-(double)(i & ~1) / (double)hidden * log_base);
    const float p = (float)((i & 1) ? cos(angle) : sin(angle));
    const float v = (ok ? Num<T>::to_f(row[i]) : 0.0f) + p;
    row_buf[i] = v;
    sum += v;
  }
  const float mean = block_sum(sum, red) / (float)hidden;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float d = row_buf[i] - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = inv_sqrt_exact(block_sum(sq, red) / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    out[(size_t)t * hidden + i] = (row_buf[i] - mean) * rstd * weight[i];
}

template <typename Kern>
int big_smem(Kern kern, size_t smem) {
  if (smem > 200 * 1024) return IFX_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

template <typename TD, typename TO>
int launch_add_layernorm(float* residual, const void* delta, int n_partials, long long partial_stride, const float* weight,
                         float eps, void* out, float* out32, const int* rows, int n_rows, int hidden, int write_residual,
                         cudaStream_t stream) {
  if (vec_ok(hidden, partial_stride, {residual, delta, weight, out, out32}))
    return launch_layernorm_vec<TD, TO, false>(residual, delta, n_partials, partial_stride, weight, eps, out, out32, rows, n_rows,
                                               hidden, write_residual, nullptr, nullptr, nullptr, nullptr, stream);
  const size_t smem = (size_t)hidden * sizeof(float);
  auto kern = add_layernorm_kernel<TD, TO>;
  int rc = big_smem(kern, smem);
  if (rc) return rc;
  rc = launch_pdl(kern, dim3(n_rows), dim3(norm_threads(hidden)), smem, stream, residual, (const TD*)delta, n_partials,
                  partial_stride, weight, eps, (TO*)out, out32, rows, hidden, write_residual);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

template <typename TD, typename TO>
int launch_add_layernorm_shift1(float* residual, const void* delta, int n_partials, long long partial_stride,
                                const float* weight, float eps, const float* mu, float* state, const int* entry_slot,
                                void* out, void* shifted, int n_rows, int hidden, cudaStream_t stream) {
  if (vec_ok(hidden, partial_stride, {residual, delta, weight, out, shifted, mu, state}))
    return launch_layernorm_vec<TD, TO, true>(residual, delta, n_partials, partial_stride, weight, eps, out, nullptr, nullptr, n_rows,
                                              hidden, 1, mu, state, entry_slot, shifted, stream);
  const size_t smem = (size_t)hidden * sizeof(float);
  auto kern = add_layernorm_shift1_kernel<TD, TO>;
  int rc = big_smem(kern, smem);
  if (rc) return rc;
  rc = launch_pdl(kern, dim3(n_rows), dim3(norm_threads(hidden)), smem, stream, residual, (const TD*)delta, n_partials,
                  partial_stride, weight, eps, mu, state, entry_slot, (TO*)out, (TO*)shifted, hidden);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
}  // namespace

// delta (null, or n_partials slices of [N, hidden], partial_stride elements apart) is added into the float32
// residual; out (out_dtype) and out32 get the normed rows; either may be null.  With rows only those rows are
// normed and the residual stays as it is.
IFX_API int ifx_add_layernorm(float* residual, const void* delta, int delta_dtype, int n_partials, long long partial_stride,
                              const float* weight, float eps, void* out, int out_dtype, float* out32, const int* rows,
                              int n_rows, int hidden, int write_residual, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (rows && write_residual) return IFX_ERR_UNSUPPORTED;
  if (n_partials < 1) n_partials = 1;
#define IFX_LN(TD, TO) return launch_add_layernorm<TD, TO>(residual, delta, n_partials, partial_stride, weight, eps, out, \
                                                           out32, rows, n_rows, hidden, write_residual, stream)
  if (delta_dtype == IFX_F32 && out_dtype == IFX_F32) IFX_LN(float, float);
  if (delta_dtype == IFX_BF16 && out_dtype == IFX_BF16) IFX_LN(bf16, bf16);
  if (delta_dtype == IFX_F32 && out_dtype == IFX_BF16) IFX_LN(float, bf16);
  if (delta_dtype == IFX_BF16 && out_dtype == IFX_F32) IFX_LN(bf16, float);
#undef IFX_LN
  return IFX_ERR_UNSUPPORTED;
}

// A step in which every entry brings one token (row t = entry t): residual sum, layer norm, token shift and
// the slot's update in one kernel.  out = the normed rows, shifted = the shifted ones, both of out_dtype.
IFX_API int ifx_add_layernorm_shift1(float* residual, const void* delta, int delta_dtype, int n_partials,
                                     long long partial_stride, const float* weight, float eps, const float* mu,
                                     float* state, const int* entry_slot, void* out, void* shifted, int out_dtype,
                                     int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (n_partials < 1) n_partials = 1;
#define IFX_LNS(TD, TO) return launch_add_layernorm_shift1<TD, TO>(residual, delta, n_partials, partial_stride, weight, eps, \
                                                                   mu, state, entry_slot, out, shifted, n_rows, hidden, stream)
  if (delta_dtype == IFX_F32 && out_dtype == IFX_F32) IFX_LNS(float, float);
  if (delta_dtype == IFX_BF16 && out_dtype == IFX_BF16) IFX_LNS(bf16, bf16);
  if (delta_dtype == IFX_F32 && out_dtype == IFX_BF16) IFX_LNS(float, bf16);
  if (delta_dtype == IFX_BF16 && out_dtype == IFX_F32) IFX_LNS(bf16, float);
#undef IFX_LNS
  return IFX_ERR_UNSUPPORTED;
}

// out[t] = h32[t] + (before(t) - h32[t]) * mu; state [slots, hidden] float32.  row_entry [N]: the entry of
// each row.
IFX_API int ifx_token_shift(const float* h32, const float* mu, float* state, const int* row_entry,
                            const int* entry_q_start, const int* entry_q_len, const int* entry_slot, void* out,
                            int out_dtype, int n_rows, int hidden, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
  int rc;
  if (out_dtype == IFX_F32)
    rc = launch_pdl(token_shift_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, h32, mu, state, row_entry,
                    entry_q_start, entry_q_len, entry_slot, (float*)out, hidden);
  else if (out_dtype == IFX_BF16)
    rc = launch_pdl(token_shift_kernel<bf16>, dim3(n_rows), dim3(threads), 0, stream, h32, mu, state, row_entry,
                    entry_q_start, entry_q_len, entry_slot, (bf16*)out, hidden);
  else
    return IFX_ERR_UNSUPPORTED;
  return rc ? rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_embed_sinusoid_layernorm(const void* table, int table_dtype, const int* ids, const int* positions,
                                         const float* weight, float eps, double base, float* out, int n_tokens,
                                         int hidden, int vocab, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (!(base > 0.0)) return IFX_ERR_UNSUPPORTED;
  const size_t smem = (size_t)hidden * sizeof(float);
  const double log_base = log(base);
  int rc;
  if (table_dtype == IFX_F32) {
    auto kern = embed_sinusoid_layernorm_kernel<float>;
    if ((rc = big_smem(kern, smem))) return rc;
    rc = launch_pdl(kern, dim3(n_tokens), dim3(norm_threads(hidden)), smem, stream, (const float*)table, ids, positions,
                    weight, eps, log_base, out, hidden, vocab);
  } else if (table_dtype == IFX_BF16) {
    auto kern = embed_sinusoid_layernorm_kernel<bf16>;
    if ((rc = big_smem(kern, smem))) return rc;
    rc = launch_pdl(kern, dim3(n_tokens), dim3(norm_threads(hidden)), smem, stream, (const bf16*)table, ids, positions,
                    weight, eps, log_base, out, hidden, vocab);
  } else {
    return IFX_ERR_UNSUPPORTED;
  }
  return rc ? rc : IFX_LAUNCH_CHECK();
}
