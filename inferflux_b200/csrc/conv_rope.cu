// A short causal convolution over time on every channel of a stacked projection, rotary positions on the
// query and key heads, and the write of keys and values into the paged cache, in one kernel:
//
//   y_t[c] = sum_{j < taps} w[c][j] * u_{t - taps + 1 + j}[c]        u = the projection's float32 sums,
//                                                                    u = 0 ahead of a sequence's first token
//   rotation of the first `rot_dims` dimensions of each query and key head, pairs either interleaved
//   (2i, 2i+1) or split in halves (i, i + rot_dims/2):  (a, b) -> (a cos - b sin,  b cos + a sin)
//   with the step's cos/sin tables [token][rot_dims/2];  values are convolved only.
//
// The last taps-1 projected rows of every sequence live in the request's state slot ("tail"), so a prompt
// may be cut anywhere: a token whose window reaches back before the step's first row reads the tail.  The
// tail is brought up to date by a second kernel after all rows have been read.  Everything is float32 up to
// the one rounding into the engine's type.  The rotation kernel alone serves mixers without a convolution
// or a paged cache (it rotates q and k of a float32 projection in place).
#include "common.cuh"

namespace {
constexpr int MAX_TAPS = 16;
enum { LAYOUT_HALF = 0, LAYOUT_INTERLEAVED = 1 };

struct ConvRope {
  const float* proj; int parts; long long part_stride; int proj_stride;   // [parts][N][proj_stride]
  const float* conv_w;        // [channels][taps] or null (no convolution)
  int taps;
  float* tail;                // [slots][taps-1][channels]
  const int* row_entry;       // [N]
  const int* entry_q_start;   // [entries]
  const int* entry_q_len;
  const int* entry_slot;
  const float* cos_t; const float* sin_t; int rot_half; int layout;
  int n_heads, n_kv, dim, vdim;
  void* q_out;                // [N][n_heads * dim]
  const int* slot_map;        // [N] page * page_size + offset, negative = do not store
  void* k_cache; void* v_cache; long long page_stride; int page_size, page_shift;
};

__device__ __forceinline__ float proj_at(const ConvRope& p, int row, int c) {
  float v = 0.0f;
  for (int s = 0; s < p.parts; ++s) v += p.proj[(size_t)s * p.part_stride + (size_t)row * p.proj_stride + c];
  return v;
}

// The convolved value of channel c for the token at row `row`, the i-th new token of its entry.
__device__ __forceinline__ float conv_at(const ConvRope& p, int row, int i, int slot, int channels, int c) {
  if (!p.conv_w) return proj_at(p, row, c);
  float y = 0.0f;
  const float* w = p.conv_w + (size_t)c * p.taps;
  for (int j = 0; j < p.taps; ++j) {
    const int m = i - (p.taps - 1) + j;            // which token of the entry, negative = before this step
    const float u = m >= 0 ? proj_at(p, row - (i - m), c)
                           : p.tail[((size_t)slot * (p.taps - 1) + (p.taps - 1 + m)) * channels + c];
    y = fmaf(w[j], u, y);
  }
  return y;
}

// The partner of dimension d under the rotation, or -1 if d does not rotate; `first` = d is the pair's first.
__device__ __forceinline__ int rot_partner(int d, int rot_half, int layout, int& pair, bool& first) {
  if (d >= 2 * rot_half) return -1;
  if (layout == LAYOUT_INTERLEAVED) { pair = d >> 1; first = !(d & 1); return d ^ 1; }
  first = d < rot_half;
  pair = first ? d : d - rot_half;
  return first ? d + rot_half : d - rot_half;
}

template <typename T>
__global__ void __launch_bounds__(256)
conv_rope_kv_write_kernel(ConvRope p) {
  pdl_enter();
  const int t = blockIdx.x;
  const int e = p.row_entry[t];
  const int i = t - p.entry_q_start[e];
  const int slot = p.entry_slot[e];
  const int cq = p.n_heads * p.dim, ck = p.n_kv * p.dim, cv = p.n_kv * p.vdim;
  const int channels = cq + ck + cv;
  const float* ct = p.cos_t + (size_t)t * p.rot_half;
  const float* st = p.sin_t + (size_t)t * p.rot_half;
  const int where = p.slot_map ? p.slot_map[t] : -1;
  const long long page = where >= 0 ? (where >> p.page_shift) : 0;
  const int off = where & (p.page_size - 1);
  for (int c = threadIdx.x; c < channels; c += blockDim.x) {
    float y = conv_at(p, t, i, slot, channels, c);
    if (c < cq + ck) {                             // a query or key channel: rotate
      const int head = c / p.dim, d = c - head * p.dim;
      int pair = 0; bool first = false;
      const int pd = rot_partner(d, p.rot_half, p.layout, pair, first);
      if (pd >= 0) {
        const float z = conv_at(p, t, i, slot, channels, head * p.dim + pd);
        const float co = ct[pair], si = st[pair];
        y = first ? y * co - z * si : y * co + z * si;
      }
      if (c < cq) {
        ((T*)p.q_out)[(size_t)t * cq + c] = Num<T>::from_f(y);
      } else if (where >= 0) {
        const int kh = head - p.n_heads;
        ((T*)p.k_cache)[(size_t)page * p.page_stride + ((size_t)kh * p.page_size + off) * p.dim + d] = Num<T>::from_f(y);
      }
    } else if (where >= 0) {
      const int cc = c - cq - ck;
      const int vh = cc / p.vdim, d = cc - vh * p.vdim;
      ((T*)p.v_cache)[(size_t)page * p.page_stride + ((size_t)vh * p.page_size + off) * p.vdim + d] = Num<T>::from_f(y);
    }
  }
}

// The same for sizes that allow 16-byte accesses (dim, vdim, the rotated dimensions and the projection's row
// length multiples of 4): a thread takes 4 neighbouring channels, reads each of the `taps` rows with one float4,
// and stores its 4 results at once.  Interleaved pairs lie inside the thread's 4 channels; pairs split in halves
// take the partner's 4 channels from a second set of loads.  The grid's second dimension cuts the channels, so
// a step of few tokens still fills the GPU.
__device__ __forceinline__ float4 proj4_at(const ConvRope& p, int row, int c) {
  float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int s = 0; s < p.parts; ++s) {
    const float4 u = *reinterpret_cast<const float4*>(p.proj + (size_t)s * p.part_stride + (size_t)row * p.proj_stride + c);
    v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
  }
  return v;
}

__device__ __forceinline__ float4 conv4_at(const ConvRope& p, int row, int i, int slot, int channels, int c) {
  if (!p.conv_w) return proj4_at(p, row, c);
  float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  const float* w = p.conv_w + (size_t)c * p.taps;
  for (int j = 0; j < p.taps; ++j) {
    const int m = i - (p.taps - 1) + j;
    const float4 u = m >= 0 ? proj4_at(p, row - (i - m), c)
                            : *reinterpret_cast<const float4*>(p.tail + ((size_t)slot * (p.taps - 1) + (p.taps - 1 + m)) * channels + c);
    y.x = fmaf(w[j], u.x, y.x);
    y.y = fmaf(w[p.taps + j], u.y, y.y);
    y.z = fmaf(w[2 * p.taps + j], u.z, y.z);
    y.w = fmaf(w[3 * p.taps + j], u.w, y.w);
  }
  return y;
}

template <typename T> __device__ __forceinline__ void store4(T* dst, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <> __device__ __forceinline__ void store4<bf16>(bf16* dst, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&lo);
  raw.y = *reinterpret_cast<unsigned*>(&hi);
  *reinterpret_cast<uint2*>(dst) = raw;
}

template <typename T>
__global__ void __launch_bounds__(128)
conv_rope_kv_write_vec_kernel(ConvRope p) {
  pdl_enter();
  const int t = blockIdx.x;
  const int e = p.row_entry[t];
  const int i = t - p.entry_q_start[e];
  const int slot = p.entry_slot[e];
  const int cq = p.n_heads * p.dim, ck = p.n_kv * p.dim, cv = p.n_kv * p.vdim;
  const int channels = cq + ck + cv;
  const float* ct = p.cos_t + (size_t)t * p.rot_half;
  const float* st = p.sin_t + (size_t)t * p.rot_half;
  const int where = p.slot_map ? p.slot_map[t] : -1;
  const long long page = where >= 0 ? (where >> p.page_shift) : 0;
  const int off = where & (p.page_size - 1);
  const int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (c >= channels) return;
  float4 y = conv4_at(p, t, i, slot, channels, c);
  if (c < cq + ck) {
    const int head = c / p.dim, d = c - head * p.dim;
    if (d < 2 * p.rot_half) {
      if (p.layout == LAYOUT_INTERLEAVED) {                // pairs (d, d + 1) and (d + 2, d + 3)
        const float c0 = ct[d >> 1], s0 = st[d >> 1], c1 = ct[(d >> 1) + 1], s1 = st[(d >> 1) + 1];
        y = make_float4(y.x * c0 - y.y * s0, y.y * c0 + y.x * s0, y.z * c1 - y.w * s1, y.w * c1 + y.z * s1);
      } else {                                             // pairs (d, d + half): the partner's 4 channels
        const bool first = d < p.rot_half;
        const int pair = first ? d : d - p.rot_half;
        const float4 z = conv4_at(p, t, i, slot, channels, head * p.dim + (first ? d + p.rot_half : d - p.rot_half));
        const float4 co = *reinterpret_cast<const float4*>(ct + pair), si = *reinterpret_cast<const float4*>(st + pair);
        y = first ? make_float4(y.x * co.x - z.x * si.x, y.y * co.y - z.y * si.y, y.z * co.z - z.z * si.z, y.w * co.w - z.w * si.w)
                  : make_float4(y.x * co.x + z.x * si.x, y.y * co.y + z.y * si.y, y.z * co.z + z.z * si.z, y.w * co.w + z.w * si.w);
      }
    }
    if (c < cq) {
      store4<T>((T*)p.q_out + (size_t)t * cq + c, y);
    } else if (where >= 0) {
      const int kh = head - p.n_heads;
      store4<T>((T*)p.k_cache + (size_t)page * p.page_stride + ((size_t)kh * p.page_size + off) * p.dim + d, y);
    }
  } else if (where >= 0) {
    const int cc = c - cq - ck;
    const int vh = cc / p.vdim, d = cc - vh * p.vdim;
    store4<T>((T*)p.v_cache + (size_t)page * p.page_stride + ((size_t)vh * p.page_size + off) * p.vdim + d, y);
  }
}

// After the rows have been read: the tail becomes the last taps-1 rows of (old tail ++ the entry's new rows).
__global__ void __launch_bounds__(256)
conv_tail_update_kernel(ConvRope p) {
  pdl_enter();
  const int e = blockIdx.x;
  const int channels = p.n_heads * p.dim + p.n_kv * p.dim + p.n_kv * p.vdim;
  const int keep = p.taps - 1;
  const int len = p.entry_q_len[e], r0 = p.entry_q_start[e];
  float* tail = p.tail + (size_t)p.entry_slot[e] * keep * channels;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    float v[MAX_TAPS];
#pragma unroll
    for (int s = 0; s < MAX_TAPS; ++s) {
      if (s >= keep) break;
      const int m = len + s;                       // index into (old tail ++ new rows)
      v[s] = m < keep ? tail[(size_t)m * channels + c] : proj_at(p, r0 + m - keep, c);
    }
#pragma unroll
    for (int s = 0; s < MAX_TAPS; ++s) {
      if (s >= keep) break;
      tail[(size_t)s * channels + c] = v[s];
    }
  }
}

// Rotation in place of `n_rot_heads` heads of width `dim` that start at column `col0` of float32 rows.
__global__ void __launch_bounds__(256)
rotate_heads_kernel(float* __restrict__ x, int row_stride, int col0, int n_rot_heads, int dim,
                    const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_half, int layout) {
  pdl_enter();
  const int t = blockIdx.x;
  float* row = x + (size_t)t * row_stride + col0;
  const float* ct = cos_t + (size_t)t * rot_half;
  const float* st = sin_t + (size_t)t * rot_half;
  for (int w = threadIdx.x; w < n_rot_heads * rot_half; w += blockDim.x) {
    const int h = w / rot_half, i = w - h * rot_half;
    const int d0 = layout == LAYOUT_INTERLEAVED ? 2 * i : i;
    const int d1 = layout == LAYOUT_INTERLEAVED ? 2 * i + 1 : i + rot_half;
    const float a = row[h * dim + d0], b = row[h * dim + d1];
    const float co = ct[i], si = st[i];
    row[h * dim + d0] = a * co - b * si;
    row[h * dim + d1] = b * co + a * si;
  }
}
}  // namespace

IFX_API int ifx_conv_rope_kv_write(const float* proj, int parts, long long part_stride, int proj_stride,
                                   const float* conv_w, int taps, float* tail,
                                   const int* row_entry, const int* entry_q_start, const int* entry_q_len,
                                   const int* entry_slot, int n_tokens, int n_entries,
                                   const float* cos_t, const float* sin_t, int rot_half, int layout,
                                   int n_heads, int n_kv, int dim, int vdim,
                                   void* q_out, int dtype, const int* slot_map, void* k_cache, void* v_cache,
                                   long long page_stride, int page_size, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (taps > MAX_TAPS || (conv_w && taps < 1) || 2 * rot_half > dim) return IFX_ERR_UNSUPPORTED;
  if (page_size <= 0 || (page_size & (page_size - 1))) return IFX_ERR_UNSUPPORTED;
  ConvRope p{proj, parts, part_stride, proj_stride, conv_w, conv_w ? taps : 1, tail, row_entry, entry_q_start, entry_q_len,
             entry_slot, cos_t, sin_t, rot_half, layout, n_heads, n_kv, dim, vdim, q_out, slot_map, k_cache, v_cache,
             page_stride, page_size, 0};
  while ((1 << p.page_shift) < page_size) ++p.page_shift;
  const int all = n_heads * dim + n_kv * dim + n_kv * vdim;
  // 16-byte accesses: sizes multiples of 4 (of 8 where the rotation pairs halves, so a thread's 4 channels stay
  // in one half and its cos/sin are 4 aligned floats), aligned pointers
  const bool vec = !(dim & 3) && !(vdim & 3) && !(proj_stride & 3) && !(part_stride & 3) &&
                   (layout == LAYOUT_INTERLEAVED ? !(rot_half & 1) : !(rot_half & 3)) && !(page_stride & 3) &&
                   !(((uintptr_t)proj | (uintptr_t)tail | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)q_out |
                      (uintptr_t)k_cache | (uintptr_t)v_cache) & 15);
  int rc;
  if (vec) {
    const dim3 grid(n_tokens, (all / 4 + 127) / 128);
    rc = dtype == IFX_BF16 ? launch_pdl(conv_rope_kv_write_vec_kernel<bf16>, grid, dim3(128), 0, stream, p)
                           : launch_pdl(conv_rope_kv_write_vec_kernel<float>, grid, dim3(128), 0, stream, p);
  } else {
    rc = dtype == IFX_BF16 ? launch_pdl(conv_rope_kv_write_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream, p)
                           : launch_pdl(conv_rope_kv_write_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, p);
  }
  if (rc) return rc;
  if (conv_w && taps > 1) {
    const int channels = n_heads * dim + n_kv * dim + n_kv * vdim;
    rc = launch_pdl(conv_tail_update_kernel, dim3(n_entries, (channels + 1023) / 1024), dim3(256), 0, stream, p);
    if (rc) return rc;
  }
  return IFX_LAUNCH_CHECK();
}

IFX_API int ifx_rotate_heads(float* x, int row_stride, int col0, int n_rot_heads, int dim, const float* cos_t,
                             const float* sin_t, int rot_half, int layout, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0 || rot_half <= 0 || n_rot_heads <= 0) return 0;
  if (2 * rot_half > dim) return IFX_ERR_UNSUPPORTED;
  const int rc = launch_pdl(rotate_heads_kernel, dim3(n_tokens), dim3(256), 0, stream, x, row_stride, col0, n_rot_heads,
                            dim, cos_t, sin_t, rot_half, layout);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
