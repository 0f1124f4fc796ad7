// Retention: linear attention with a fixed decay per head, no softmax and no denominator,
//
//   S_t = g S_{t-1} + k_t v_t^T          S: [dim x vdim] per head, float32, in the request's state slot
//   o_t = S_t^T q_t                      g = the head's decay, k already scaled
//
// so o_t = g^(i+1) S_start^T q_t + sum_{j <= i} g^(i-j) (q_t . k_j) v_j for the i-th token of a segment that
// starts from S_start.  A portion is cut into segments of IFX_RETENTION_SEGMENT tokens that run side by side:
//   1. every segment's own sum B = sum_j g^(n-1-j) k_j v_j^T                              (segment_sums)
//   2. per entry and head the segments' starting states one after the other, S <- g^n S + B; the last one
//      goes into the slot                                                                 (carry)
//   3. every segment's outputs from its starting state                                    (outputs)
// A step whose entries all fit one segment (single tokens, short portions) runs 3 alone: it reads the slot
// and writes the new state itself.  A block owns a tile of 64 value columns of one (segment, head); the
// state tile, the segment's q, k, v and the decayed scores live in shared memory.  All of it is float32
// FFMA: the state, what enters it and the scores are 32-bit by the mixer's definition.
// `finish` divides each head's output by its root mean square, multiplies by silu(gate) and rounds once.
#include "common.cuh"

#define IFX_RETENTION_SEGMENT 32

namespace {
constexpr int SEG = IFX_RETENTION_SEGMENT;
constexpr int VT = 64;                 // value columns per block
constexpr int THREADS = 256;
constexpr int GROUPS = THREADS / VT;   // 4 groups of threads over tokens or state rows
constexpr int TPT = SEG / GROUPS;      // tokens per thread in the output step

struct RetStep {
  const float* proj; int stride;       // [N][stride] float32, q and k already rotated
  int q_col, k_col, v_col;             // first column of q, k, v (heads side by side, dim / vdim wide)
  int heads, dim, vdim;
  const float* decay;                  // [heads]
  float k_scale;
  const int* seg_entry; const int* seg_t0;
  const int* entry_q_start; const int* entry_q_len; const int* entry_slot;
  float* state;                        // [slots][heads][dim][vdim]
};

__device__ __forceinline__ void decay_powers(float* pw, float g, int tid) {
  if (tid <= SEG) pw[tid] = (float)pow((double)g, (double)tid);
}

// Rows of k in shared memory are `key_ld(dim)` floats apart: dim + 4 where dim is a multiple of 4 (rows stay
// 16-byte aligned for the vector paths and neighbouring rows fall into different banks), else dim + 1.
__host__ __device__ __forceinline__ int key_ld(int dim) { return (dim & 3) ? dim + 1 : dim + 4; }

// k[j][d] (scaled), v[j][c] for the block's columns
__device__ __forceinline__ void load_kv(const RetStep& s, int row0, int n, int head, int v0, float* ks, float* vs, int tid) {
  const int D = s.dim, KD = key_ld(D);
  for (int idx = tid; idx < SEG * D; idx += THREADS) {
    const int j = idx / D, d = idx - j * D;
    ks[j * KD + d] = j < n ? s.proj[(size_t)(row0 + j) * s.stride + s.k_col + head * D + d] * s.k_scale : 0.0f;
  }
  for (int idx = tid; idx < SEG * VT; idx += THREADS) {
    const int j = idx / VT, c = idx - j * VT;
    vs[idx] = (j < n && v0 + c < s.vdim) ? s.proj[(size_t)(row0 + j) * s.stride + s.v_col + head * s.vdim + v0 + c] : 0.0f;
  }
}

// new[d][c] = g^n old[d][c] + sum_j g^(n-1-j) k_j[d] v_j[c] for the block's columns; old may be null (zero)
__device__ __forceinline__ void fold_segment(const float* ks, const float* vs, const float* pw, int n, int D, int V, int v0,
                                             const float* old_tile /* smem [D][VT] or null */, float* dst /* global [D][V] */,
                                             int tid) {
  const int KD = key_ld(D);
  if (!(D & 3)) {
    // a thread owns 4 columns and groups of 4 state rows: per token one 16-byte load of keys and one of values
    const int cg = tid & 15, dg = tid >> 4;
    for (int grp = dg; grp < D / 4; grp += THREADS / 16) {
      float acc[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
      for (int j = 0; j < n; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks + j * KD + 4 * grp);
        const float4 v4 = *reinterpret_cast<const float4*>(vs + j * VT + 4 * cg);
        const float w = pw[n - 1 - j];
        const float kk[4] = {k4.x * w, k4.y * w, k4.z * w, k4.w * w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(kk[a], vv[b], acc[a][b]);
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int d = 4 * grp + a;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int c = 4 * cg + b;
          if (v0 + c < V) dst[(size_t)d * V + v0 + c] = old_tile ? fmaf(pw[n], old_tile[d * VT + c], acc[a][b]) : acc[a][b];
        }
      }
    }
    return;
  }
  const int c = tid % VT, g = tid / VT;
  if (v0 + c >= V) return;
  for (int d = g; d < D; d += GROUPS) {
    float acc = old_tile ? pw[n] * old_tile[d * VT + c] : 0.0f;
    for (int j = 0; j < n; ++j) acc = fmaf(pw[n - 1 - j] * ks[j * KD + d], vs[j * VT + c], acc);
    dst[(size_t)d * V + v0 + c] = acc;
  }
}

__global__ void __launch_bounds__(THREADS)
retention_segment_sums_kernel(RetStep s, float* __restrict__ seg_b) {
  pdl_enter();
  extern __shared__ float smem[];
  const int D = s.dim, V = s.vdim;
  float* ks = smem;                        // [SEG][key_ld(D)]
  float* vs = ks + SEG * key_ld(D);        // [SEG][VT]
  float* pw = vs + SEG * VT;               // [SEG + 1]
  const int seg = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * VT, tid = threadIdx.x;
  const int e = s.seg_entry[seg], t0 = s.seg_t0[seg];
  const int n = min(SEG, s.entry_q_len[e] - t0);
  decay_powers(pw, s.decay[head], tid);
  load_kv(s, s.entry_q_start[e] + t0, n, head, v0, ks, vs, tid);
  __syncthreads();
  fold_segment(ks, vs, pw, n, D, V, v0, nullptr, seg_b + ((size_t)seg * s.heads + head) * D * V, tid);
}

__global__ void __launch_bounds__(THREADS)
retention_carry_kernel(RetStep s, const int* __restrict__ entry_first_seg, const float* __restrict__ seg_b,
                       float* __restrict__ seg_start) {
  pdl_enter();
  const int e = blockIdx.x, head = blockIdx.y;
  const size_t tile = (size_t)s.dim * s.vdim;
  const int len = s.entry_q_len[e];
  const int n_seg = (len + SEG - 1) / SEG, seg0 = entry_first_seg[e];
  const double g = (double)s.decay[head];
  const float g_full = (float)pow(g, (double)SEG), g_last = (float)pow(g, (double)(len - (n_seg - 1) * SEG));
  float* st = s.state + ((size_t)s.entry_slot[e] * s.heads + head) * tile;
  for (size_t at = (size_t)blockIdx.z * THREADS + threadIdx.x; at < tile; at += (size_t)gridDim.z * THREADS) {
    float S = st[at];
    const size_t step = (size_t)s.heads * tile;
    const size_t o0 = ((size_t)seg0 * s.heads + head) * tile + at;
    for (int k0 = 0; k0 < n_seg; k0 += 8) {        // eight segments' sums are asked for before the first is used
      float bs[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) bs[u] = k0 + u < n_seg ? seg_b[o0 + (size_t)(k0 + u) * step] : 0.0f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int k = k0 + u;
        if (k >= n_seg) break;
        seg_start[o0 + (size_t)k * step] = S;
        S = fmaf(k == n_seg - 1 ? g_last : g_full, S, bs[u]);
      }
    }
    st[at] = S;
  }
}

// seg_start: the segments' starting states from the carry, or null: every entry is one segment, the state
// comes from the slot and goes back there.
__global__ void __launch_bounds__(THREADS)
retention_outputs_kernel(RetStep s, const float* __restrict__ seg_start, float* __restrict__ out /* [N][heads * vdim] */) {
  pdl_enter();
  extern __shared__ float smem[];
  const int D = s.dim, V = s.vdim;
  const int KD = key_ld(D);
  float* ks = smem;                        // [SEG][KD]
  float* vs = ks + SEG * KD;               // [SEG][VT]
  float* pw = vs + SEG * VT;               // [SEG + 1] (+ padding to a multiple of 4)
  float* qs = pw + SEG + 4;                // [SEG][D]
  float* St = qs + SEG * D;                // [D][VT]
  float* P = St + D * VT;                  // [SEG][SEG + 1]
  const int seg = blockIdx.x, head = blockIdx.y, v0 = blockIdx.z * VT, tid = threadIdx.x;
  const int e = s.seg_entry[seg], t0 = s.seg_t0[seg];
  const int n = min(SEG, s.entry_q_len[e] - t0);
  const int row0 = s.entry_q_start[e] + t0;
  decay_powers(pw, s.decay[head], tid);
  load_kv(s, row0, n, head, v0, ks, vs, tid);
  for (int idx = tid; idx < SEG * D; idx += THREADS) {
    const int j = idx / D, d = idx - j * D;
    qs[idx] = j < n ? s.proj[(size_t)(row0 + j) * s.stride + s.q_col + head * D + d] : 0.0f;
  }
  float* slot_tile = s.state + ((size_t)s.entry_slot[e] * s.heads + head) * D * V;
  const float* start = seg_start ? seg_start + ((size_t)seg * s.heads + head) * D * V : slot_tile;
  for (int idx = tid; idx < D * VT; idx += THREADS) {
    const int d = idx / VT, c = idx - d * VT;
    St[idx] = v0 + c < V ? start[(size_t)d * V + v0 + c] : 0.0f;
  }
  __syncthreads();
  // decayed scores of the segment: P[i][j] = g^(i-j) (q_i . k_j) for j <= i
  if (!(D & 3)) {
    // a thread takes rows bi, bi + 16 against keys bj, bj + 16: four dot products from 16-byte loads
    const int bi = tid >> 4, bj = tid & 15;
    float d00 = 0.0f, d01 = 0.0f, d10 = 0.0f, d11 = 0.0f;
    for (int d = 0; d < D; d += 4) {
      const float4 qa = *reinterpret_cast<const float4*>(qs + bi * D + d), qb = *reinterpret_cast<const float4*>(qs + (bi + 16) * D + d);
      const float4 ka = *reinterpret_cast<const float4*>(ks + bj * KD + d), kb = *reinterpret_cast<const float4*>(ks + (bj + 16) * KD + d);
      d00 = fmaf(qa.x, ka.x, fmaf(qa.y, ka.y, fmaf(qa.z, ka.z, fmaf(qa.w, ka.w, d00))));
      d01 = fmaf(qa.x, kb.x, fmaf(qa.y, kb.y, fmaf(qa.z, kb.z, fmaf(qa.w, kb.w, d01))));
      d10 = fmaf(qb.x, ka.x, fmaf(qb.y, ka.y, fmaf(qb.z, ka.z, fmaf(qb.w, ka.w, d10))));
      d11 = fmaf(qb.x, kb.x, fmaf(qb.y, kb.y, fmaf(qb.z, kb.z, fmaf(qb.w, kb.w, d11))));
    }
    const int i0 = bi, i1 = bi + 16, j0 = bj, j1 = bj + 16;
    P[i0 * (SEG + 1) + j0] = (j0 <= i0 && i0 < n) ? d00 * pw[i0 - j0] : 0.0f;
    P[i0 * (SEG + 1) + j1] = 0.0f;                                   // j1 >= 16 > i0
    P[i1 * (SEG + 1) + j0] = i1 < n ? d10 * pw[i1 - j0] : 0.0f;      // j0 < 16 <= i1
    P[i1 * (SEG + 1) + j1] = (j1 <= i1 && i1 < n) ? d11 * pw[i1 - j1] : 0.0f;
  } else {
    for (int idx = tid; idx < SEG * SEG; idx += THREADS) {
      const int i = idx / SEG, j = idx - i * SEG;
      float dot = 0.0f;
      if (j <= i && i < n) {
        const float* qa = qs + i * D;
        const float* kb = ks + j * KD;
        for (int d = 0; d < D; ++d) dot = fmaf(qa[d], kb[d], dot);
        dot *= pw[i - j];
      }
      P[i * (SEG + 1) + j] = dot;
    }
  }
  __syncthreads();
  if (!(D & 3)) {
    // a thread owns tokens tg, tg + 16 and 4 columns: per 4 state rows four 16-byte loads of the state and two of q
    const int cg = tid & 15, tg = tid >> 4;
    float inter[2][4], intra[2][4];
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) { inter[a][b] = 0.0f; intra[a][b] = 0.0f; }
    for (int d = 0; d < D; d += 4) {
      const float4 qa = *reinterpret_cast<const float4*>(qs + tg * D + d), qb = *reinterpret_cast<const float4*>(qs + (tg + 16) * D + d);
      const float qv[2][4] = {{qa.x, qa.y, qa.z, qa.w}, {qb.x, qb.y, qb.z, qb.w}};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float4 s4 = *reinterpret_cast<const float4*>(St + (d + u) * VT + 4 * cg);
        const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int b = 0; b < 4; ++b) inter[a][b] = fmaf(qv[a][u], sv[b], inter[a][b]);
      }
    }
    for (int j = 0; j < n; ++j) {
      const float4 v4 = *reinterpret_cast<const float4*>(vs + j * VT + 4 * cg);
      const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
      const float pa = P[tg * (SEG + 1) + j], pb = P[(tg + 16) * (SEG + 1) + j];
#pragma unroll
      for (int b = 0; b < 4; ++b) { intra[0][b] = fmaf(pa, vv[b], intra[0][b]); intra[1][b] = fmaf(pb, vv[b], intra[1][b]); }
    }
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      const int i = tg + 16 * a;
      if (i >= n) continue;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int c = 4 * cg + b;
        if (v0 + c < V) out[(size_t)(row0 + i) * s.heads * V + (size_t)head * V + v0 + c] = fmaf(pw[i + 1], inter[a][b], intra[a][b]);
      }
    }
  } else {
    const int c = tid % VT, g = tid / VT;
    float inter[TPT], intra[TPT];
#pragma unroll
    for (int u = 0; u < TPT; ++u) { inter[u] = 0.0f; intra[u] = 0.0f; }
    for (int d = 0; d < D; ++d) {
      const float sv = St[d * VT + c];
#pragma unroll
      for (int u = 0; u < TPT; ++u) inter[u] = fmaf(qs[(g + GROUPS * u) * D + d], sv, inter[u]);
    }
    for (int j = 0; j < n; ++j) {
      const float vv = vs[j * VT + c];
#pragma unroll
      for (int u = 0; u < TPT; ++u) intra[u] = fmaf(P[(g + GROUPS * u) * (SEG + 1) + j], vv, intra[u]);
    }
    if (v0 + c < V) {
#pragma unroll
      for (int u = 0; u < TPT; ++u) {
        const int i = g + GROUPS * u;
        if (i < n) out[(size_t)(row0 + i) * s.heads * V + (size_t)head * V + v0 + c] = fmaf(pw[i + 1], inter[u], intra[u]);
      }
    }
  }
  if (!seg_start) fold_segment(ks, vs, pw, n, D, V, v0, St, slot_tile, tid);   // every thread writes only what it read
}

// out[t][h][:] = o[t][h][:] / sqrt(mean(o^2) + eps) * silu(gate[t][h][:]); a warp per (token, head)
template <typename T>
__global__ void __launch_bounds__(256)
retention_finish_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_stride, T* __restrict__ out,
                        long long out_stride, int n_tokens, int heads, int vdim, float eps) {
  pdl_enter();
  const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (w >= n_tokens * heads) return;
  const int t = w / heads, h = w - t * heads;
  const float* row = o + ((size_t)t * heads + h) * vdim;
  float ss = 0.0f;
  for (int d = lane; d < vdim; d += 32) ss = fmaf(row[d], row[d], ss);
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
  const float* gr = gate + (size_t)t * gate_stride + (size_t)h * vdim;
  T* orow = out + (size_t)t * out_stride + (size_t)h * vdim;
  for (int d = lane; d < vdim; d += 32) {
    const float gv = gr[d];
    orow[d] = Num<T>::from_f(row[d] * inv * (gv / (1.0f + expf(-gv))));
  }
}

size_t outputs_smem(int D) {
  return ((size_t)SEG * key_ld(D) + SEG * VT + SEG + 4 + (size_t)SEG * D + (size_t)D * VT + SEG * (SEG + 1)) * sizeof(float);
}
}  // namespace

IFX_API int ifx_retention_segment() { return SEG; }

// proj: float32 [N][stride] with q, k (rotated) and v at the given columns.  multi = some entry has more than
// one segment: then seg_b and seg_start ([segments][heads][dim][vdim] float32 each) are used.
IFX_API int ifx_retention_scan(const float* proj, int stride, int q_col, int k_col, int v_col, int heads, int dim, int vdim,
                               const float* decay, float k_scale, float* state,
                               const int* seg_entry, const int* seg_t0, int n_segments, const int* entry_first_seg,
                               const int* entry_q_start, const int* entry_q_len, const int* entry_slot, int n_entries,
                               int multi, float* seg_b, float* seg_start, float* out, cudaStream_t stream) {
  if (n_segments <= 0) return 0;
  if (dim < 1 || dim > 256 || vdim < 1 || heads < 1 || heads > 65535) return IFX_ERR_UNSUPPORTED;
  RetStep s{proj, stride, q_col, k_col, v_col, heads, dim, vdim, decay, k_scale, seg_entry, seg_t0, entry_q_start,
            entry_q_len, entry_slot, state};
  const int vtiles = (vdim + VT - 1) / VT;
  const size_t smem_c = outputs_smem(dim);
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(retention_outputs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)outputs_smem(256));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(retention_segment_sums_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  int rc;
  if (multi) {
    const size_t smem_a = ((size_t)SEG * key_ld(dim) + SEG * VT + SEG + 4) * sizeof(float);
    rc = launch_pdl(retention_segment_sums_kernel, dim3(n_segments, heads, vtiles), dim3(THREADS), smem_a, stream, s, seg_b);
    if (rc) return rc;
    const int zb = (int)(((size_t)dim * vdim + 4 * THREADS - 1) / (4 * THREADS));
    rc = launch_pdl(retention_carry_kernel, dim3(n_entries, heads, zb), dim3(THREADS), 0, stream, s, entry_first_seg,
                    (const float*)seg_b, seg_start);
    if (rc) return rc;
  }
  rc = launch_pdl(retention_outputs_kernel, dim3(n_segments, heads, vtiles), dim3(THREADS), smem_c, stream, s,
                  (const float*)(multi ? seg_start : nullptr), out);
  return rc ? rc : IFX_LAUNCH_CHECK();
}

IFX_API int ifx_retention_finish(const float* o, const float* gate, int gate_stride, void* out, int out_dtype,
                                 long long out_stride, int n_tokens, int heads, int vdim, float eps, cudaStream_t stream) {
  const int warps = n_tokens * heads;
  if (warps <= 0) return 0;
  const dim3 grid((warps + 7) / 8);
  const int rc = out_dtype == IFX_BF16
      ? launch_pdl(retention_finish_kernel<bf16>, grid, dim3(256), 0, stream, o, gate, gate_stride, (bf16*)out, out_stride, n_tokens, heads, vdim, eps)
      : launch_pdl(retention_finish_kernel<float>, grid, dim3(256), 0, stream, o, gate, gate_stride, (float*)out, out_stride, n_tokens, heads, vdim, eps);
  return rc ? rc : IFX_LAUNCH_CHECK();
}
