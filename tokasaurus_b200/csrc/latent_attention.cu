// Attention over a cache of per-token latents ("latent attention"): every token leaves one row
// [c (rank) | rotated shared key part (rot)] in its request's pages, and all query heads read the same rows.
// With the key up-projection folded into the query (q_abs = W_uk^T q_plain, done by the caller as a matrix
// product), a head's score for a key row is  (q_abs . c + q_rot . k_rot) * scale,  and its output in latent
// space is the softmax-weighted sum of the rows' c, which the caller takes through the value up-projection.
//
// Kernels: the preparation of a step's tokens (RMS norms of the query latent and of c, interleaved rotation of the
// shared key part, write into the pages); the interleaved rotation of the queries' rotated part; the attention
// itself on the FP32 pipes for any mix of prompt portions and single tokens (scores, softmax weights and sums
// float32).  Each is built for float and bfloat16 activations.
//
// Both rotations also come in the other pairing (halves: channel i with channel i + rot_dims / 2), with frequencies
// given in float64 (freq64: the angle, its sine and cosine are then made in float64, once a token) and with a factor
// `mag` on every sine and cosine (a frequency-scaling scheme's attention factor).  head_sigmoid_gate multiplies every
// head's output by the sigmoid of a per-token, per-head logit (an output gate).
//
// Compile with -DTKB_LAT_RANK=<rank of the latent>.
#include "common.cuh"
#include <float.h>

#ifndef TKB_LAT_RANK
#error "compile with -DTKB_LAT_RANK=<rank of the cached latent>"
#endif

using namespace tkb;

namespace {

constexpr int RANK = TKB_LAT_RANK;
constexpr int WARPS = 4;
constexpr int DPL = (RANK + 31) / 32;  // output elements per lane

// ------------------------------------------------------------------------------------------------
// One block a token.  proj: float32 [tokens, stride] holding the query latent at column q_off (q_rank wide, absent
// if q_rank == 0) and the key/value latent at column kv_off (RANK + rot wide, absent if kv_off < 0).
//   cq = rms(proj[q_off : q_off + q_rank]) * q_w                          -> cq_out [tokens, q_rank]
//   c  = rms(proj[kv_off : kv_off + RANK]) * kv_w                         -> cache row [0, RANK)
//   kr = rotate(proj[kv_off + RANK : + rot], position)                    -> cache row [RANK, RANK + rot)
// The rotation turns the pairs (2i, 2i+1), i < rot_dims / 2, by position * inv_freq[i]; the rest passes.
template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ proj, int stride, int q_off, int q_rank,
                                   const float* __restrict__ q_w, T* __restrict__ cq_out, int kv_off, int rot,
                                   int rot_dims, const float* __restrict__ kv_w, const float* __restrict__ inv_freq,
                                   T* __restrict__ cache, const int* __restrict__ positions,
                                   const int* __restrict__ token_seq, const int* __restrict__ page_indptr,
                                   const int* __restrict__ page_ids, int page_size, int num_pages, float eps,
                                   int* __restrict__ status, const double* __restrict__ freq64, int halves, float mag) {
  __shared__ float scratch[33];
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  if (s < 0) return;
  const float* row = proj + (size_t)t * stride;
  if (q_rank > 0) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) ss += row[q_off + i] * row[q_off + i];
    const float r = rsqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
      cq_out[(size_t)t * q_rank + i] = from_float<T>(row[q_off + i] * r * q_w[i]);
  }
  if (kv_off < 0) return;
  const int p = positions[t];
  const int page = checked_page(page_ids[page_indptr[s] + p / page_size], num_pages, status);
  float ss = 0.f;
  for (int i = threadIdx.x; i < RANK; i += blockDim.x) ss += row[kv_off + i] * row[kv_off + i];
  const float r = rsqrtf(block_sum(ss, scratch) / (float)RANK + eps);
  if (page < 0) {
    if (threadIdx.x == 0) atomicOr(status, TKB_STATUS_BAD_PAGE);
    return;
  }
  T* dst = cache + ((size_t)page * page_size + (p % page_size)) * (RANK + rot);
  for (int i = threadIdx.x; i < RANK; i += blockDim.x) dst[i] = from_float<T>(row[kv_off + i] * r * kv_w[i]);
  const float* kr = row + kv_off + RANK;
  const int half = rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    if (freq64 != nullptr) {
      double s64, c64;
      sincos((double)p * freq64[i], &s64, &c64);
      sn = (float)s64 * mag;
      cs = (float)c64 * mag;
    } else {
      sincosf((float)p * inv_freq[i], &sn, &cs);
    }
    const int a = halves ? i : 2 * i, b = halves ? i + half : 2 * i + 1;
    const float u = kr[a], v = kr[b];
    dst[RANK + a] = from_float<T>(u * cs - v * sn);
    dst[RANK + b] = from_float<T>(v * cs + u * sn);
  }
  for (int i = rot_dims + threadIdx.x; i < rot; i += blockDim.x) dst[RANK + i] = from_float<T>(kr[i]);
}

// dst[t][head][dst_off + i] = rotated src[t][head][src_off + i], i < rot: the pairs (2i, 2i+1), i < rot_dims / 2, are
// turned by position * inv_freq[i], the values from rot_dims on pass unchanged.  dst may be src (in place).
constexpr int ROT_TABLE = 256;  // most rotated pairs of a head

template <typename T>
__global__ void rotate_pairs_kernel(const T* __restrict__ src, int src_token_stride, int src_head_stride, int src_off,
                                    T* __restrict__ dst, int dst_token_stride, int dst_head_stride, int dst_off,
                                    int n_heads, int rot, int rot_dims, const float* __restrict__ inv_freq,
                                    const int* __restrict__ positions, const int* __restrict__ token_seq,
                                    const double* __restrict__ freq64, int halves, float mag) {
  __shared__ float tcs[ROT_TABLE], tsn[ROT_TABLE];
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  if (token_seq[t] < 0) return;
  const int half = rot_dims / 2, per_head = half + (rot - rot_dims);
  // the token's cosines and sines once, for all heads
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    if (freq64 != nullptr) {
      double s64, c64;
      sincos((double)positions[t] * freq64[i], &s64, &c64);
      tsn[i] = (float)s64 * mag;
      tcs[i] = (float)c64 * mag;
    } else {
      sincosf((float)positions[t] * inv_freq[i], &tsn[i], &tcs[i]);
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_heads * per_head; idx += blockDim.x) {
    const int h = idx / per_head, i = idx - h * per_head;
    const T* q = src + (size_t)t * src_token_stride + (size_t)h * src_head_stride + src_off;
    T* o = dst + (size_t)t * dst_token_stride + (size_t)h * dst_head_stride + dst_off;
    if (i < half) {
      const int a = halves ? i : 2 * i, b = halves ? i + half : 2 * i + 1;
      const float sn = tsn[i], cs = tcs[i];
      const float u = to_float(q[a]), v = to_float(q[b]);
      o[a] = from_float<T>(u * cs - v * sn);
      o[b] = from_float<T>(v * cs + u * sn);
    } else {
      o[rot_dims + i - half] = q[rot_dims + i - half];
    }
  }
}

// val[r][h][:] *= sigmoid(gate[token(r)][gate_off + h]): an output gate, one number a (token, head); gate float32 with
// row stride gate_stride; rows names the tokens that val's rows belong to (null: row r is token r).  One block a row.
template <typename T>
__global__ void head_sigmoid_gate_kernel(T* __restrict__ val, const float* __restrict__ gate, int gate_stride,
                                         int gate_off, const int* __restrict__ rows, int n_heads, int vdim) {
  trigger_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const float* g = gate + (size_t)(rows ? rows[r] : r) * gate_stride + gate_off;
  for (int idx = threadIdx.x; idx < n_heads * vdim; idx += blockDim.x) {
    const float f = 1.f / (1.f + expf(-g[idx / vdim]));
    val[(size_t)r * n_heads * vdim + idx] = from_float<T>(to_float(val[(size_t)r * n_heads * vdim + idx]) * f);
  }
}

// ------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float dot_span(const T* __restrict__ k, const float* __restrict__ q, int n, bool vec);

template <>
__device__ __forceinline__ float dot_span<float>(const float* __restrict__ k, const float* __restrict__ q, int n,
                                                 bool vec) {
  float acc = 0.f;
  if (vec) {
    const float4* k4 = reinterpret_cast<const float4*>(k);
    for (int i = 0; i < n / 4; i++) {
      const float4 v = k4[i];
      acc = fmaf(v.x, q[4 * i + 0], acc);
      acc = fmaf(v.y, q[4 * i + 1], acc);
      acc = fmaf(v.z, q[4 * i + 2], acc);
      acc = fmaf(v.w, q[4 * i + 3], acc);
    }
    return acc;
  }
  for (int i = 0; i < n; i++) acc = fmaf(k[i], q[i], acc);
  return acc;
}
template <>
__device__ __forceinline__ float dot_span<__nv_bfloat16>(const __nv_bfloat16* __restrict__ k,
                                                         const float* __restrict__ q, int n, bool vec) {
  float acc = 0.f;
  if (vec) {
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
    for (int i = 0; i < n / 8; i++) {
      const uint4 v = k8[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const float2 f = __bfloat1622float2(h[u]);
        acc = fmaf(f.x, q[8 * i + 2 * u + 0], acc);
        acc = fmaf(f.y, q[8 * i + 2 * u + 1], acc);
      }
    }
    return acc;
  }
  for (int i = 0; i < n; i++) acc = fmaf(__bfloat162float(k[i]), q[i], acc);
  return acc;
}

// One warp owns one (token, head).  A token at position p sees the rows of positions max(0, p - window + 1) .. p of
// its own request (window <= 0: all); the step's own rows are in the cache already.  Lane j scores row base + j;
// after the warp-wide running maximum and sum are brought up to date, lane d accumulates latent elements d, d + 32, ...
// splits > 1 (steps of few rows, which would leave most SMs idle): the visible rows of a (token, head) are shared out
// among blockIdx.z warps in runs of a multiple of 32 rows; each leaves its sums, maximum (log2 units) and weight sum in
// part[((row * heads + head) * splits + split) * (RANK + 2)], and latent_attn_merge puts them together.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
latent_attn_simt_kernel(const T* __restrict__ q_abs, long long qa_token_stride, long long qa_head_stride,
                        const T* __restrict__ q_rot, long long qr_token_stride, long long qr_head_stride, int rot,
                        T* __restrict__ out, const T* __restrict__ cache, const int* __restrict__ token_seq,
                        const int* __restrict__ positions, const int* __restrict__ page_indptr,
                        const int* __restrict__ page_ids, const int* __restrict__ rows, int n_heads, int page_size,
                        float scale_log2, int window, int num_pages, int* __restrict__ status, int splits,
                        float* __restrict__ part) {
  extern __shared__ float qs_all[];  // [WARPS][RANK + rot]
  trigger_dependents();
  grid_dependency_wait();
  const int t = rows ? rows[blockIdx.x] : blockIdx.x;
  const int s = token_seq[t];
  if (s < 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = blockIdx.y * WARPS + warp;
  if (h >= n_heads) return;
  const int width = RANK + rot;
  float* qs = qs_all + (size_t)warp * width;
  const int p = positions[t];
  const int* table = page_ids + page_indptr[s];
  int lo = 0;
  if (window > 0 && p - window + 1 > 0) lo = p - window + 1;
  const T* qa = q_abs + (size_t)t * qa_token_stride + (size_t)h * qa_head_stride;
  const T* qr = q_rot + (size_t)t * qr_token_stride + (size_t)h * qr_head_stride;
  for (int d = lane; d < RANK; d += 32) qs[d] = to_float(qa[d]) * scale_log2;
  for (int d = lane; d < rot; d += 32) qs[RANK + d] = to_float(qr[d]) * scale_log2;
  __syncwarp();
  const bool vec = (width * sizeof(T)) % 16 == 0;

  float m = -FLT_MAX, l = 0.f;
  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; i++) acc[i] = 0.f;
  int first = lo, last = p;
  if (splits > 1) {
    const int per = (((p - lo + 1) + splits - 1) / splits + 31) & ~31;
    first = lo + (int)blockIdx.z * per;
    last = min(p, first + per - 1);
  }
  for (int base = first; base <= last; base += 32) {
    const int j = base + lane;
    const bool live = j <= last;
    long long rowoff = 0;
    float sc = -FLT_MAX;
    if (live) {
      const int page = checked_page(table[j / page_size], num_pages, status);
      if (page >= 0) {
        rowoff = ((long long)page * page_size + (j % page_size)) * width;
        sc = dot_span<T>(cache + rowoff, qs, width, vec);
      }
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float alpha = exp2f(m - m_new);
    const float pj = (live && sc > -FLT_MAX) ? exp2f(sc - m_new) : 0.f;
    l = l * alpha + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int i = 0; i < DPL; i++) acc[i] *= alpha;
    const int nlive = (last - base + 1) < 32 ? (last - base + 1) : 32;
    for (int jj = 0; jj < nlive; jj++) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const long long ro = __shfl_sync(0xffffffffu, rowoff, jj);
      const T* crow = cache + ro;
#pragma unroll
      for (int i = 0; i < DPL; i++) {
        const int d = lane + 32 * i;
        if (d < RANK) acc[i] = fmaf(pv, to_float(crow[d]), acc[i]);
      }
    }
  }
  if (splits > 1) {
    float* pr = part + (((size_t)blockIdx.x * n_heads + h) * splits + blockIdx.z) * (RANK + 2);
#pragma unroll
    for (int i = 0; i < DPL; i++) {
      const int d = lane + 32 * i;
      if (d < RANK) pr[d] = acc[i];
    }
    if (lane == 0) {
      pr[RANK] = m;
      pr[RANK + 1] = l;
    }
    return;
  }
  const float inv_l = l > 0.f ? 1.f / l : 0.f;
  T* orow = out + ((size_t)blockIdx.x * n_heads + h) * RANK;
#pragma unroll
  for (int i = 0; i < DPL; i++) {
    const int d = lane + 32 * i;
    if (d < RANK) orow[d] = from_float<T>(acc[i] * inv_l);
  }
}

// The shares of a (row, head) put together: grid (rows, heads).
template <typename T>
__global__ void latent_attn_merge_kernel(const float* __restrict__ part, T* __restrict__ out, int n_heads, int splits) {
  trigger_dependents();
  grid_dependency_wait();
  const float* pr = part + ((size_t)blockIdx.x * n_heads + blockIdx.y) * splits * (RANK + 2);
  float mm = -FLT_MAX;
  for (int z = 0; z < splits; z++) mm = fmaxf(mm, pr[z * (RANK + 2) + RANK]);
  float ll = 0.f;
  for (int z = 0; z < splits; z++) ll += exp2f(pr[z * (RANK + 2) + RANK] - mm) * pr[z * (RANK + 2) + RANK + 1];
  const float inv = ll > 0.f ? 1.f / ll : 0.f;
  for (int d = threadIdx.x; d < RANK; d += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < splits; z++) acc += exp2f(pr[z * (RANK + 2) + RANK] - mm) * pr[z * (RANK + 2) + d];
    out[((size_t)blockIdx.x * n_heads + blockIdx.y) * RANK + d] = from_float<T>(acc * inv);
  }
}

template <typename T>
int prep_launch(const float* proj, int stride, int q_off, int q_rank, const float* q_w, void* cq_out, int kv_off,
                int rot, int rot_dims, const float* kv_w, const float* inv_freq, void* cache, const int* positions,
                const int* token_seq, const int* page_indptr, const int* page_ids, int page_size, int num_pages,
                float eps, int n_tokens, int* status, const double* freq64, int halves, float mag, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (rot_dims < 0 || rot_dims > rot || rot_dims % 2 || page_size <= 0) return -2;
  return launch_pdl(latent_prep_kernel<T>, dim3(n_tokens), dim3(128), 0, st, proj, stride, q_off, q_rank, q_w,
                    (T*)cq_out, kv_off, rot, rot_dims, kv_w, inv_freq, (T*)cache, positions, token_seq, page_indptr,
                    page_ids, page_size, num_pages, eps, status, freq64, halves, mag);
}

template <typename T>
int rotate_launch(const void* src, int src_ts, int src_hs, int src_off, void* dst, int dst_ts, int dst_hs, int dst_off,
                  int n_heads, int rot, int rot_dims, const float* inv_freq, const int* positions, const int* token_seq,
                  int n_tokens, const double* freq64, int halves, float mag, cudaStream_t st) {
  if (n_tokens <= 0 || rot <= 0) return 0;
  if (rot_dims % 2 || rot_dims > rot || rot_dims / 2 > ROT_TABLE) return -2;
  return launch_pdl(rotate_pairs_kernel<T>, dim3(n_tokens), dim3(128), 0, st, (const T*)src, src_ts, src_hs, src_off,
                    (T*)dst, dst_ts, dst_hs, dst_off, n_heads, rot, rot_dims, inv_freq, positions, token_seq, freq64,
                    halves, mag);
}

template <typename T>
int attn_launch(const void* q_abs, long long qa_ts, long long qa_hs, const void* q_rot, long long qr_ts, long long qr_hs,
                int rot, void* out, const void* cache, const int* token_seq, const int* positions,
                const int* page_indptr, const int* page_ids, const int* rows, int n_rows, int n_heads, int page_size,
                float scale, int window, int num_pages, int* status, int splits, float* part, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (n_heads <= 0 || page_size <= 0 || rot < 0) return -2;
  if (splits < 1 || part == nullptr) splits = 1;
  if (splits > 64 || n_heads > 65535) return -2;
  const int hb = (n_heads + WARPS - 1) / WARPS;
  if (hb > 65535) return -3;
  const size_t smem = (size_t)WARPS * (RANK + rot) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_attn_simt_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int rc = launch_pdl(latent_attn_simt_kernel<T>, dim3(n_rows, hb, splits), dim3(WARPS * 32), smem, st, (const T*)q_abs,
                      qa_ts, qa_hs, (const T*)q_rot, qr_ts, qr_hs, rot, (T*)out, (const T*)cache, token_seq, positions,
                      page_indptr, page_ids, rows, n_heads, page_size, scale * 1.4426950408889634f, window, num_pages,
                      status, splits, part);
  if (rc != 0 || splits == 1) return rc;
  return launch_pdl(latent_attn_merge_kernel<T>, dim3(n_rows, n_heads), dim3(RANK >= 128 ? 128 : 64), 0, st,
                    (const float*)part, (T*)out, n_heads, splits);
}

}  // namespace

#define TKB_LATENT_EXPORTS(SUF, T)                                                                                     \
  TKB_EXPORT int tkb_latent_prep_##SUF(const float* proj, int stride, int q_off, int q_rank, const float* q_w,         \
                                       void* cq_out, int kv_off, int rot, int rot_dims, const float* kv_w,             \
                                       const float* inv_freq, void* cache, const int* positions, const int* token_seq, \
                                       const int* page_indptr, const int* page_ids, int page_size, int num_pages,      \
                                       float eps, int n_tokens, int* status, const double* freq64, int halves,         \
                                       float mag, void* st) {                                                          \
    return prep_launch<T>(proj, stride, q_off, q_rank, q_w, cq_out, kv_off, rot, rot_dims, kv_w, inv_freq, cache,      \
                          positions, token_seq, page_indptr, page_ids, page_size, num_pages, eps, n_tokens, status,    \
                          freq64, halves, mag, (cudaStream_t)st);                                                      \
  }                                                                                                                    \
  TKB_EXPORT int tkb_head_sigmoid_gate_##SUF(void* val, const float* gate, int gate_stride, int gate_off,              \
                                             const int* rows, int n_rows, int n_heads, int vdim, void* st) {           \
    if (n_rows <= 0) return 0;                                                                                         \
    if (n_heads <= 0 || vdim <= 0) return -2;                                                                          \
    return launch_pdl(head_sigmoid_gate_kernel<T>, dim3(n_rows), dim3(256), 0, (cudaStream_t)st, (T*)val, gate,        \
                      gate_stride, gate_off, rows, n_heads, vdim);                                                     \
  }                                                                                                                    \
  TKB_EXPORT int tkb_rotate_pairs_##SUF(const void* src, int src_ts, int src_hs, int src_off, void* dst, int dst_ts,    \
                                        int dst_hs, int dst_off, int n_heads, int rot, int rot_dims,                   \
                                        const float* inv_freq, const int* positions, const int* token_seq,             \
                                        int n_tokens, const double* freq64, int halves, float mag, void* st) {         \
    return rotate_launch<T>(src, src_ts, src_hs, src_off, dst, dst_ts, dst_hs, dst_off, n_heads, rot, rot_dims,        \
                            inv_freq, positions, token_seq, n_tokens, freq64, halves, mag, (cudaStream_t)st);          \
  }                                                                                                                    \
  TKB_EXPORT int tkb_latent_attn_simt_##SUF(const void* q_abs, long long qa_ts, long long qa_hs, const void* q_rot,    \
                                            long long qr_ts, long long qr_hs, int rot, void* out, const void* cache,   \
                                            const int* token_seq, const int* positions, const int* page_indptr,        \
                                            const int* page_ids, const int* rows, int n_rows, int n_heads,             \
                                            int page_size, float scale, int window, int num_pages, int* status,        \
                                            int splits, float* part, void* st) {                                       \
    return attn_launch<T>(q_abs, qa_ts, qa_hs, q_rot, qr_ts, qr_hs, rot, out, cache, token_seq, positions,             \
                          page_indptr, page_ids, rows, n_rows, n_heads, page_size, scale, window, num_pages, status,   \
                          splits, part, (cudaStream_t)st);                                                             \
  }

TKB_LATENT_EXPORTS(f32, float)
TKB_LATENT_EXPORTS(bf16, __nv_bfloat16)
TKB_EXPORT int tkb_latent_rank() { return RANK; }
