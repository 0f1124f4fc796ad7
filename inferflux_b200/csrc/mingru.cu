// minGRU: a gated recurrence whose gates read only the current token.
//
//   z_t = sigmoid(pz_t)        pz, pu, pg: the float32 sums of the stacked projection [z | x | g] of a token
//   c_t = pu_t + 1/2  (pu_t >= 0),  sigmoid(pu_t)  (pu_t < 0)
//   S_t = (1 - z_t) S_{t-1} + z_t c_t            element by element, float32, S_{-1} = the request's state slot
//   y_t = S_t * silu(pg_t)
//
// The recurrence is linear in S, S_t = a_t S_{t-1} + b_t, so a portion is cut into segments of up to
// IFX_MINGRU_SEGMENT tokens that run side by side:
//   1. every segment finds its own (A, B) = (product of a, the recurrence from zero)
//   2. per entry the segments' starting states follow one after the other from the slot's: S <- A S + B
//   3. every segment runs the recurrence again from its starting state and writes y; the last one of an
//      entry leaves its S in the slot.
// A step whose entries all fit one segment (single tokens, short portions) runs 3 alone, from the slot.
// A thread owns one channel; channels are independent.
#include "common.cuh"

#define IFX_MINGRU_SEGMENT 32

namespace {
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

struct GruStep {
  const float* proj;          // [N, 3 * width]
  const float* bias;          // [2 * width]: the biases of z and of x, or null
  const int* seg_entry;       // [segments]
  const int* seg_t0;          // [segments] first token of the segment within its entry
  const int* entry_q_start;   // [entries]
  const int* entry_q_len;
  const int* entry_slot;
  int width;
};

__device__ __forceinline__ void gate(const float* row, int width, int ch, float bz, float bx, float& a, float& b) {
  const float z = sigmoid_f(row[ch] + bz);
  const float u = row[width + ch] + bx;
  const float c = u >= 0.0f ? u + 0.5f : sigmoid_f(u);
  a = 1.0f - z;
  b = z * c;
}

__global__ void __launch_bounds__(128)
mingru_segment_sums_kernel(GruStep s, float* __restrict__ seg_a, float* __restrict__ seg_b) {
  pdl_enter();
  const int seg = blockIdx.x, ch = blockIdx.y * blockDim.x + threadIdx.x;
  if (ch >= s.width) return;
  const int e = s.seg_entry[seg], t0 = s.seg_t0[seg];
  const int n = min(IFX_MINGRU_SEGMENT, s.entry_q_len[e] - t0);
  const float* row = s.proj + (size_t)(s.entry_q_start[e] + t0) * 3 * s.width;
  const float bz = s.bias ? s.bias[ch] : 0.0f, bx = s.bias ? s.bias[s.width + ch] : 0.0f;
  float A = 1.0f, B = 0.0f;
#pragma unroll 8
  for (int t = 0; t < n; ++t, row += 3 * s.width) {
    float a, b;
    gate(row, s.width, ch, bz, bx, a, b);
    A *= a;
    B = fmaf(a, B, b);
  }
  seg_a[(size_t)seg * s.width + ch] = A;
  seg_b[(size_t)seg * s.width + ch] = B;
}

__global__ void __launch_bounds__(128)
mingru_carry_kernel(GruStep s, const int* __restrict__ entry_first_seg, const float* __restrict__ seg_a,
                    const float* __restrict__ seg_b, const float* __restrict__ state, float* __restrict__ seg_start) {
  pdl_enter();
  const int e = blockIdx.x, ch = blockIdx.y * blockDim.x + threadIdx.x;
  if (ch >= s.width) return;
  const int n_seg = (s.entry_q_len[e] + IFX_MINGRU_SEGMENT - 1) / IFX_MINGRU_SEGMENT;
  const int seg0 = entry_first_seg[e];
  float S = state[(size_t)s.entry_slot[e] * s.width + ch];
  for (int k = 0; k < n_seg; ++k) {
    const size_t at = (size_t)(seg0 + k) * s.width + ch;
    seg_start[at] = S;
    S = fmaf(seg_a[at], S, seg_b[at]);
  }
}

template <typename TO>
__global__ void __launch_bounds__(128)
mingru_scan_kernel(GruStep s, const float* __restrict__ seg_start, float* __restrict__ state, TO* __restrict__ out,
                   long long out_stride) {
  pdl_enter();
  const int seg = blockIdx.x, ch = blockIdx.y * blockDim.x + threadIdx.x;
  if (ch >= s.width) return;
  const int e = s.seg_entry[seg], t0 = s.seg_t0[seg];
  const int len = s.entry_q_len[e];
  const int n = min(IFX_MINGRU_SEGMENT, len - t0);
  const size_t row0 = (size_t)(s.entry_q_start[e] + t0);
  const float* row = s.proj + row0 * 3 * s.width;
  TO* o = out + row0 * out_stride + ch;
  float* st = state + (size_t)s.entry_slot[e] * s.width + ch;
  const float bz = s.bias ? s.bias[ch] : 0.0f, bx = s.bias ? s.bias[s.width + ch] : 0.0f;
  float S = seg_start ? seg_start[(size_t)seg * s.width + ch] : *st;
#pragma unroll 8
  for (int t = 0; t < n; ++t, row += 3 * s.width, o += out_stride) {
    float a, b;
    gate(row, s.width, ch, bz, bx, a, b);
    S = fmaf(a, S, b);
    const float g = row[2 * s.width + ch];
    *o = Num<TO>::from_f(S * (g * sigmoid_f(g)));
  }
  if (t0 + n == len) *st = S;
}
}  // namespace

IFX_API int ifx_mingru_segment() { return IFX_MINGRU_SEGMENT; }

// proj float32 [N, 3 * width]; bias float32 [2 * width] (of z and x) or null; state float32 [slots, width]; out
// [N, width] of out_dtype, rows out_stride elements apart.  The segments of the
// step are listed by seg_entry / seg_t0 (an entry's segments in order, entry_first_seg[e] the index of its
// first).  multi != 0: some entry has more than one segment, and scratch holds 3 * n_segments * width floats.
IFX_API int ifx_mingru_scan(const float* proj, const float* bias, float* state, void* out, long long out_stride, int out_dtype, const int* seg_entry,
                            const int* seg_t0, int n_segments, const int* entry_first_seg, const int* entry_q_start,
                            const int* entry_q_len, const int* entry_slot, int n_entries, int width, int multi,
                            float* scratch, cudaStream_t stream) {
  if (n_segments <= 0 || width <= 0) return 0;
  GruStep s{proj, bias, seg_entry, seg_t0, entry_q_start, entry_q_len, entry_slot, width};
  const int threads = 128, cols = (width + threads - 1) / threads;
  if (cols > 65535) return IFX_ERR_UNSUPPORTED;
  int rc;
  float* seg_start = nullptr;
  if (multi) {
    if (!scratch) return IFX_ERR_UNSUPPORTED;
    float* seg_a = scratch;
    float* seg_b = scratch + (size_t)n_segments * width;
    seg_start = scratch + (size_t)2 * n_segments * width;
    rc = launch_pdl(mingru_segment_sums_kernel, dim3(n_segments, cols), dim3(threads), 0, stream, s, seg_a, seg_b);
    if (rc) return rc;
    rc = launch_pdl(mingru_carry_kernel, dim3(n_entries, cols), dim3(threads), 0, stream, s, entry_first_seg,
                    (const float*)seg_a, (const float*)seg_b, (const float*)state, seg_start);
    if (rc) return rc;
  }
  if (out_dtype == IFX_F32)
    rc = launch_pdl(mingru_scan_kernel<float>, dim3(n_segments, cols), dim3(threads), 0, stream, s, (const float*)seg_start,
                    state, (float*)out, out_stride);
  else if (out_dtype == IFX_BF16)
    rc = launch_pdl(mingru_scan_kernel<bf16>, dim3(n_segments, cols), dim3(threads), 0, stream, s, (const float*)seg_start,
                    state, (bf16*)out, out_stride);
  else
    return IFX_ERR_UNSUPPORTED;
  return rc ? rc : IFX_LAUNCH_CHECK();
}
