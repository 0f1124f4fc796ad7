// PolyNorm activation of a feed-forward:  y = a N(z) + b N(z^2) + c N(z^3) + e  with powers taken element by
// element and N(v) = v / sqrt(mean(v^2) + eps) over a token's row; z = the up projection's float32 sums plus
// its bias.  One block per row; the row stays in shared memory between the sums and the output.  The three
// mean squares and the result are float32; the output is rounded once to the engine's type.
#include "common.cuh"

namespace {
template <typename TO>
__global__ void polynorm_kernel(const float* __restrict__ z, long long z_stride, const float* __restrict__ bias,
                                const float* __restrict__ coeff, float eps, TO* __restrict__ out, long long out_stride, int n) {
  pdl_enter();
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  const float* zr = z + (size_t)blockIdx.x * z_stride;
  float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = zr[i] + (bias ? bias[i] : 0.0f);
    row_buf[i] = v;
    const float v2 = v * v, v3 = v2 * v;
    s1 = fmaf(v, v, s1);
    s2 = fmaf(v2, v2, s2);
    s3 = fmaf(v3, v3, s3);
  }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  s3 = block_sum(s3, red);
  const float r1 = coeff[0] / sqrtf(s1 / (float)n + eps);
  const float r2 = coeff[1] / sqrtf(s2 / (float)n + eps);
  const float r3 = coeff[2] / sqrtf(s3 / (float)n + eps);
  const float e = coeff[3];
  TO* o = out + (size_t)blockIdx.x * out_stride;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = row_buf[i];
    const float v2 = v * v;
    o[i] = Num<TO>::from_f(fmaf(v, r1, fmaf(v2, r2, fmaf(v2 * v, r3, e))));
  }
}

// The same with 16-byte loads and 8-byte stores: n a multiple of 4, rows and bias on 16-byte boundaries.
template <typename TO>
__global__ void polynorm_vec_kernel(const float* __restrict__ z, long long z_stride, const float* __restrict__ bias,
                                    const float* __restrict__ coeff, float eps, TO* __restrict__ out, long long out_stride, int n) {
  pdl_enter();
  extern __shared__ float4 row_buf4[];
  __shared__ float red[32];
  const float4* zr = reinterpret_cast<const float4*>(z + (size_t)blockIdx.x * z_stride);
  const float4* b4 = reinterpret_cast<const float4*>(bias);
  const int groups = n >> 2;
  float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
  for (int i = threadIdx.x; i < groups; i += blockDim.x) {
    float4 v = zr[i];
    if (bias) { const float4 b = b4[i]; v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
    row_buf4[i] = v;
    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float v2 = e[k] * e[k], v3 = v2 * e[k];
      s1 = fmaf(e[k], e[k], s1);
      s2 = fmaf(v2, v2, s2);
      s3 = fmaf(v3, v3, s3);
    }
  }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  s3 = block_sum(s3, red);
  const float r1 = coeff[0] / sqrtf(s1 / (float)n + eps);
  const float r2 = coeff[1] / sqrtf(s2 / (float)n + eps);
  const float r3 = coeff[2] / sqrtf(s3 / (float)n + eps);
  const float e0 = coeff[3];
  TO* o = out + (size_t)blockIdx.x * out_stride;
  for (int i = threadIdx.x; i < groups; i += blockDim.x) {
    const float4 v = row_buf4[i];
    float y[4];
    const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float v2 = e[k] * e[k];
      y[k] = fmaf(e[k], r1, fmaf(v2, r2, fmaf(v2 * e[k], r3, e0)));
    }
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(o)[i] = make_float4(y[0], y[1], y[2], y[3]);
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(y[0], y[1]), b = __floats2bfloat162_rn(y[2], y[3]);
      uint2 u;
      u.x = *reinterpret_cast<unsigned*>(&a);
      u.y = *reinterpret_cast<unsigned*>(&b);
      reinterpret_cast<uint2*>(o)[i] = u;
    }
  }
}

// Long rows (n a multiple of 4, 16-byte boundaries): 1,024 threads a row, thread t holds the groups of four elements
// t, t + 1,024, ... in registers between the three sums and the output, so a row is read once and written once.
template <typename TO, int J>
__global__ void __launch_bounds__(1024)
polynorm_reg_kernel(const float* __restrict__ z, long long z_stride, const float* __restrict__ bias,
                    const float* __restrict__ coeff, float eps, TO* __restrict__ out, long long out_stride, int n) {
  pdl_enter();
  __shared__ float red[32];
  const float4* zr = reinterpret_cast<const float4*>(z + (size_t)blockIdx.x * z_stride);
  const float4* b4 = reinterpret_cast<const float4*>(bias);
  const int groups = n >> 2;
  float4 v[J];
  float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int gi = threadIdx.x + j * 1024;
    if (gi < groups) {
      float4 x = zr[gi];
      if (bias) { const float4 b = b4[gi]; x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w; }
      v[j] = x;
      const float e[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float v2 = e[k] * e[k], v3 = v2 * e[k];
        s1 = fmaf(e[k], e[k], s1);
        s2 = fmaf(v2, v2, s2);
        s3 = fmaf(v3, v3, s3);
      }
    }
  }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  s3 = block_sum(s3, red);
  const float r1 = coeff[0] / sqrtf(s1 / (float)n + eps);
  const float r2 = coeff[1] / sqrtf(s2 / (float)n + eps);
  const float r3 = coeff[2] / sqrtf(s3 / (float)n + eps);
  const float e0 = coeff[3];
  TO* o = out + (size_t)blockIdx.x * out_stride;
#pragma unroll
  for (int j = 0; j < J; ++j) {
    const int gi = threadIdx.x + j * 1024;
    if (gi < groups) {
      const float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
      float y[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float v2 = e[k] * e[k];
        y[k] = fmaf(e[k], r1, fmaf(v2, r2, fmaf(v2 * e[k], r3, e0)));
      }
      if constexpr (sizeof(TO) == 4) {
        reinterpret_cast<float4*>(o)[gi] = make_float4(y[0], y[1], y[2], y[3]);
      } else {
        __nv_bfloat162 a = __floats2bfloat162_rn(y[0], y[1]), b = __floats2bfloat162_rn(y[2], y[3]);
        uint2 u;
        u.x = *reinterpret_cast<unsigned*>(&a);
        u.y = *reinterpret_cast<unsigned*>(&b);
        reinterpret_cast<uint2*>(o)[gi] = u;
      }
    }
  }
}

template <typename TO>
int launch_polynorm_reg(const float* z, long long z_stride, const float* bias, const float* coeff, float eps, void* out,
                        long long out_stride, int n_rows, int n, cudaStream_t stream) {
  int rc = IFX_ERR_UNSUPPORTED;
#define IFX_PN(J) case J: rc = launch_pdl(polynorm_reg_kernel<TO, J>, dim3(n_rows), dim3(1024), 0, stream, z, z_stride, bias, coeff, \
                                          eps, (TO*)out, out_stride, n); break;
  switch ((n / 4 + 1023) / 1024) {
    IFX_PN(1) IFX_PN(2) IFX_PN(3) IFX_PN(4) IFX_PN(5) IFX_PN(6) IFX_PN(7) IFX_PN(8)
    default: return IFX_ERR_UNSUPPORTED;
  }
#undef IFX_PN
  return rc ? rc : IFX_LAUNCH_CHECK();
}
}  // namespace

// z float32 [rows, n] (row stride z_stride), bias float32 [n] or null, coeff float32 [4] = a, b, c, e.
IFX_API int ifx_polynorm(const float* z, long long z_stride, const float* bias, const float* coeff, float eps, void* out,
                         long long out_stride, int out_dtype, int n_rows, int n, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const size_t smem = (size_t)n * sizeof(float);
  if (smem > 200 * 1024) return IFX_ERR_UNSUPPORTED;
  int threads = 64;
  while (threads < 1024 && threads * 4 < n) threads <<= 1;
  int rc;
  const bool vec = n % 4 == 0 && (z_stride & 3) == 0 && (out_stride & 3) == 0 && (((uintptr_t)z | (uintptr_t)bias | (uintptr_t)out) & 15) == 0;
  if (vec && n >= 2048 && n <= 4 * 8 * 1024) {           // the row length alone decides which kernel sums a row
    if (out_dtype == IFX_F32) return launch_polynorm_reg<float>(z, z_stride, bias, coeff, eps, out, out_stride, n_rows, n, stream);
    if (out_dtype == IFX_BF16) return launch_polynorm_reg<bf16>(z, z_stride, bias, coeff, eps, out, out_stride, n_rows, n, stream);
  }
  if (vec && (out_dtype == IFX_F32 || out_dtype == IFX_BF16)) {
    threads = 64;
    while (threads < 1024 && threads * 8 < n) threads <<= 1;
    if (out_dtype == IFX_F32) {
      auto kern = polynorm_vec_kernel<float>;
      if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return (int)cudaGetLastError();
      rc = launch_pdl(kern, dim3(n_rows), dim3(threads), smem, stream, z, z_stride, bias, coeff, eps, (float*)out, out_stride, n);
    } else {
      auto kern = polynorm_vec_kernel<bf16>;
      if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return (int)cudaGetLastError();
      rc = launch_pdl(kern, dim3(n_rows), dim3(threads), smem, stream, z, z_stride, bias, coeff, eps, (bf16*)out, out_stride, n);
    }
    return rc ? rc : IFX_LAUNCH_CHECK();
  }
  if (out_dtype == IFX_F32) {
    auto kern = polynorm_kernel<float>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return (int)cudaGetLastError();
    rc = launch_pdl(kern, dim3(n_rows), dim3(threads), smem, stream, z, z_stride, bias, coeff, eps, (float*)out, out_stride, n);
  } else if (out_dtype == IFX_BF16) {
    auto kern = polynorm_kernel<bf16>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return (int)cudaGetLastError();
    rc = launch_pdl(kern, dim3(n_rows), dim3(threads), smem, stream, z, z_stride, bias, coeff, eps, (bf16*)out, out_stride, n);
  } else {
    return IFX_ERR_UNSUPPORTED;
  }
  return rc ? rc : IFX_LAUNCH_CHECK();
}
