// Two small operations on the float32 residual stream, for blocks that rewrite it between layers.
//   add_into:         r[t, :] += sum_p d[p][t, :]          (the slices added in index order)
//   add_rows_vector:  out[t, :] = a[t, :] + b[t, :] + v[:]
#include "common.cuh"

namespace {
template <typename TD>
__global__ void add_into_kernel(float* __restrict__ r, const TD* __restrict__ d, int n_partials, long long partial_stride,
                                long long total) {
  pdl_enter();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float v = r[i];
    for (int p = 0; p < n_partials; ++p) v += Num<TD>::to_f(d[i + (long long)p * partial_stride]);
    r[i] = v;
  }
}

__global__ void add_rows_vector_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ v,
                                       float* __restrict__ out, int hidden, long long total) {
  pdl_enter();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    out[i] = a[i] + b[i] + v[i % hidden];
}

int grid_for(long long total) {
  long long blocks = (total + 255) / 256;
  return (int)(blocks < 1 ? 1 : (blocks > 4096 ? 4096 : blocks));
}
}  // namespace

IFX_API int ifx_add_into(float* r, const void* d, int d_dtype, int n_partials, long long partial_stride, long long total,
                         cudaStream_t stream) {
  if (total <= 0) return 0;
  if (n_partials < 1) n_partials = 1;
  int rc;
  if (d_dtype == IFX_F32)
    rc = launch_pdl(add_into_kernel<float>, dim3(grid_for(total)), dim3(256), 0, stream, r, (const float*)d, n_partials,
                    partial_stride, total);
  else if (d_dtype == IFX_BF16)
    rc = launch_pdl(add_into_kernel<bf16>, dim3(grid_for(total)), dim3(256), 0, stream, r, (const bf16*)d, n_partials,
                    partial_stride, total);
  else
    return IFX_ERR_UNSUPPORTED;
  return rc ? rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_add_rows_vector(const float* a, const float* b, const float* v, float* out, int n_rows, int hidden,
                                cudaStream_t stream) {
  const long long total = (long long)n_rows * hidden;
  if (total <= 0) return 0;
  const int rc = launch_pdl(add_rows_vector_kernel, dim3(grid_for(total)), dim3(256), 0, stream, a, b, v, out, hidden, total);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
