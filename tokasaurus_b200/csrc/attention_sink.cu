// Grouped-query attention over the paged cache with a soft cap on the scores and a per-head sink in the softmax, for
// heads whose keys and values have different sizes:
//
//     s_ij = cap * tanh(scale * q_i . k_j / cap)   (cap <= 0: s_ij = scale * q_i . k_j),
//     o_i  = sum_j exp(s_ij) v_j / (exp(sink_h) + sum_j exp(s_ij)),      j over max(0, i - window + 1) .. i
//
// The sink takes part in the denominator only: it has no key and no value.  sink == null: an ordinary softmax.
// A cached row holds one token's key and value of one key/value head side by side: [k (QK values) | v (VD values)],
// rows [page][kv head][slot in page][QK + VD].
//
// Two kernels.  sink_attn_prep: one block a token; adds the projections' biases, divides every q head and every k
// head by its root mean square (float32, no weight) if asked, writes q in the activation type and the token's
// [k | v] rows into its page.  attn_sink_simt: one warp a (token, query head) on the FP32 pipes, any mix of prompt
// portions and single tokens; lane j scores key base + j, probabilities are passed round by shuffle while lane d
// sums output elements d, d + 32, ...  Scores, weights and sums are float32.
//
//
// In bfloat16, for key and value sizes that are multiples of 16 up to 256, two tensor-core kernels
// (mma.sync m16n8k16, float32 scores, weights rounded to bfloat16 for their product with the values) take the place of
// the FP32-pipe kernel.  Both stage 64 cached rows at a time in shared memory (cp.async, two buffers; a row's key and
// value arrive in one copy) and keep a running softmax that the sink opens.  attn_sink_tiles: a block owns 64 queries
// of one request's portion and one query head, a warp 16 of them.  attn_sink_single: a block owns a request that
// brings one token and one key/value head; the MMA rows are that head's query heads, the four warps take every
// fourth group of 16 keys and are merged through shared memory; with few requests a request's tiles are shared out
// among several blocks and a small kernel puts their shares together.  Blocks find their work from the step's request
// table themselves, so a launch depends on the step's shape only.
//
// A second weight function, chosen at compile time (-DTKB_SIGMOID=1): no softmax, the weight of a visible key is
// sigmoid(s_ij), not normalised over the keys (no sink, no running maximum; partial sums of blocks and warps simply add).
// In both forms a head may carry a factor on its scale and a number added to its scores (head_scale, head_bias:
// float32 [heads] or null): s_ij = cap(scale * head_scale_h * q_i . k_j) + head_bias_h.
//
// sink_attn_prep can also scale the normed q and k heads by weight vectors, rotate them by position (pairs of
// neighbouring channels or of the two halves of the first rot_dims channels; angles, sines and cosines float64, made
// once a token), and cache the key as projected (before norm and rotation) as the value (values_are_keys: QK == VD, the
// projections hold no v).
//
// Several attention maps a head (-DTKB_MAPS=2): q holds heads * MAPS query vectors, head by head [map 0, map 1, ...], the
// projections as many key vectors a key/value head, and a cached row is [k of map 0 | k of map 1 | ... | v].  Every map
// is an attention of its own over the same values; the kernels treat (head, map) as a query head whose keys start
// MAP * QK values into the row, and leave the maps' outputs side by side in float32 [rows, heads, MAPS, VD] (what
// combines them wants them unrounded).  diff_combine (MAPS == 2) is the differential form's combination:
// o = a_0 - lambda a_1, divided by its root mean square over VD, times a number and the sigmoid of a per-head gate.
//
// keep_first: with a window, the first keep_first positions of a request stay visible to every later query
// (position i sees j if j <= i and (i - j < window or j < keep_first)).
//
// Compile with -DTKB_QK=<query/key size> -DTKB_VD=<value size> [-DTKB_SIGMOID=1] [-DTKB_MAPS=2].
#include "common.cuh"
#include <float.h>
#include <type_traits>

#if !defined(TKB_QK) || !defined(TKB_VD)
#error "compile with -DTKB_QK=<query/key size> -DTKB_VD=<value size>"
#endif
static_assert(TKB_QK >= 1 && TKB_QK <= 512 && TKB_VD >= 1 && TKB_VD <= 512, "head sizes up to 512");
#ifndef TKB_SIGMOID
#define TKB_SIGMOID 0
#endif
#ifndef TKB_MAPS
#define TKB_MAPS 1
#endif
static_assert(TKB_MAPS >= 1 && TKB_MAPS <= 4, "one to four attention maps a head");

using namespace tkb;

namespace {

constexpr int QK = TKB_QK;
constexpr int VD = TKB_VD;
constexpr int MAPS = TKB_MAPS;
constexpr int KW = MAPS * QK;  // key values of a cached row; the value follows them
constexpr int ROW = KW + VD;
constexpr int WARPS = 4;
constexpr int DPL = (VD + 31) / 32;
constexpr bool SIGMOID = TKB_SIGMOID != 0;

template <typename T>
__device__ __forceinline__ float dot_key(const T* __restrict__ k, const float* __restrict__ q) {
  float acc = 0.f;
  if constexpr (sizeof(T) == 4 && QK % 4 == 0 && ROW % 4 == 0) {
    const float4* k4 = reinterpret_cast<const float4*>(k);
#pragma unroll 8
    for (int i = 0; i < QK / 4; i++) {
      const float4 v = k4[i];
      acc = fmaf(v.x, q[4 * i + 0], acc);
      acc = fmaf(v.y, q[4 * i + 1], acc);
      acc = fmaf(v.z, q[4 * i + 2], acc);
      acc = fmaf(v.w, q[4 * i + 3], acc);
    }
  } else if constexpr (sizeof(T) == 2 && QK % 8 == 0 && ROW % 8 == 0) {
    const uint4* k8 = reinterpret_cast<const uint4*>(k);
#pragma unroll 4
    for (int i = 0; i < QK / 8; i++) {
      const uint4 v = k8[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const float2 f = __bfloat1622float2(h[u]);
        acc = fmaf(f.x, q[8 * i + 2 * u + 0], acc);
        acc = fmaf(f.y, q[8 * i + 2 * u + 1], acc);
      }
    }
  } else {
#pragma unroll 8
    for (int i = 0; i < QK; i++) acc = fmaf(to_float(k[i]), q[i], acc);
  }
  return acc;
}

// qkv: float32 [T, stride] = [q (nh * QK) | k (nkv * QK) | v (nkv * VD)]  (no v if values_are_keys)
// norm_w: float32 [2][QK] weights of the q heads' and the k heads' norm, or null; freq: float64 [rot_dims / 2] or null
template <typename T>
__global__ void __launch_bounds__(256)
sink_attn_prep_kernel(const float* __restrict__ qkv, int stride, const float* __restrict__ bias, int unit_norm,
                      float eps, T* __restrict__ q_out, T* __restrict__ cache, const int* __restrict__ positions,
                      const int* __restrict__ token_seq, const int* __restrict__ page_indptr,
                      const int* __restrict__ page_ids, int nh, int nkv, int page_size, int num_pages, int write_cache,
                      int* __restrict__ status, const float* __restrict__ norm_w, const double* __restrict__ freq,
                      int rot_dims, int rot_pairs, int values_are_keys) {
  __shared__ float rot_cs[QK];  // [rot_dims / 2] cosines, then as many sines
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  if (s < 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const float* row = qkv + (size_t)t * stride;
  const int p = positions[t];
  int page = -1;
  if (write_cache) page = checked_page(page_ids[page_indptr[s] + p / page_size], num_pages, status);
  const int slot = p % page_size;
  const int half = freq != nullptr ? rot_dims / 2 : 0;
  if (half > 0) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      double sn, cs;
      sincos((double)p * freq[i], &sn, &cs);
      rot_cs[i] = (float)cs;
      rot_cs[half + i] = (float)sn;
    }
    __syncthreads();
  }
  // q vectors and k vectors (MAPS of each a head): one warp a vector
  const int nhq = nh * MAPS, nkk = nkv * MAPS;
  for (int hh = warp; hh < nhq + nkk; hh += nwarps) {
    const int off = hh * QK;  // the k vectors follow the q vectors in the row
    float ss = 0.f;
    for (int d = lane; d < QK; d += 32) {
      const float v = row[off + d] + (bias ? bias[off + d] : 0.f);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float r = unit_norm ? rsqrtf(ss / (float)QK + eps) : 1.f;
    T* dst = nullptr;
    if (hh < nhq) dst = q_out + (size_t)t * nhq * QK + off;
    else if (page >= 0)
      dst = cache + (((size_t)page * nkv + (hh - nhq) / MAPS) * page_size + slot) * ROW + ((hh - nhq) % MAPS) * QK;
    if (dst != nullptr) {
      const float* w = norm_w ? norm_w + (hh < nhq ? 0 : QK) : nullptr;
      auto val = [&](int d) { return (row[off + d] + (bias ? bias[off + d] : 0.f)) * r * (w ? w[d] : 1.f); };
      for (int i = lane; i < half; i += 32) {
        const int a = rot_pairs ? 2 * i : i, b = rot_pairs ? 2 * i + 1 : i + half;
        const float u = val(a), v = val(b), c = rot_cs[i], sn = rot_cs[half + i];
        dst[a] = from_float<T>(u * c - v * sn);
        dst[b] = from_float<T>(v * c + u * sn);
      }
      for (int d = 2 * half + lane; d < QK; d += 32) dst[d] = from_float<T>(val(d));
    }
  }
  if (page >= 0) {
    const int voff = values_are_keys ? nhq * QK : (nhq + nkk) * QK;  // the keys as projected are the values
    for (int idx = threadIdx.x; idx < nkv * VD; idx += blockDim.x) {
      const int g = idx / VD, d = idx - g * VD;
      cache[(((size_t)page * nkv + g) * page_size + slot) * ROW + KW + d] =
          from_float<T>(row[voff + idx] + (bias ? bias[voff + idx] : 0.f));
    }
  }
}

// With several maps a head the maps' outputs stay float32 (they are combined before anything rounds them).
template <typename T> struct OutOf { using type = typename std::conditional<(MAPS > 1), float, T>::type; };

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_sink_simt_kernel(const T* __restrict__ q, typename OutOf<T>::type* __restrict__ out, const T* __restrict__ cache,
                      const int* __restrict__ token_seq, const int* __restrict__ positions,
                      const int* __restrict__ page_indptr, const int* __restrict__ page_ids,
                      const int* __restrict__ rows, const float* __restrict__ sinks, int nh, int nkv, int page_size,
                      float scale, float softcap, int window, int keep_first, int num_pages, int* __restrict__ status,
                      const float* __restrict__ head_scale, const float* __restrict__ head_bias) {
  using TO = typename OutOf<T>::type;
  __shared__ float qs[WARPS][QK];
  trigger_dependents();
  grid_dependency_wait();
  const int t = rows ? rows[blockIdx.x] : blockIdx.x;
  const int kvh = blockIdx.y;
  const int s = token_seq[t];
  if (s < 0) return;
  const int p = positions[t];
  const int group = nh / nkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int* table = page_ids + page_indptr[s];
  int lo = 0;
  if (window > 0 && p - window + 1 > 0) lo = p - window + 1;
  // the positions kept in sight before the window: [0, kept)
  const int kept = (window > 0 && keep_first > 0) ? min(keep_first, lo) : 0;
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;

  for (int gq = warp; gq < group * MAPS; gq += WARPS) {
    const int h = kvh * group * MAPS + gq;  // (head, map) counted as a query head
    const int koff = (gq % MAPS) * QK;
    const T* qrow = q + ((size_t)t * nh * MAPS + h) * QK;
    for (int d = lane; d < QK; d += 32) qs[warp][d] = to_float(qrow[d]);
    __syncwarp();

    const float hscale = scale * (head_scale ? head_scale[h] : 1.f), hbias = head_bias ? head_bias[h] : 0.f;
    // the sink opens the running softmax: maximum sink, sum exp(sink - sink) = 1, nothing accumulated
    float m = sinks ? sinks[h] : -FLT_MAX;
    float l = sinks ? 1.f : 0.f;
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; i++) acc[i] = 0.f;

    for (int seg = (kept > 0 ? 0 : 1); seg < 2; seg++) {
      const int first = seg == 0 ? 0 : lo, last = seg == 0 ? kept - 1 : p;
      for (int base = first; base <= last; base += 32) {
        const int j = base + lane;
        const bool live = j <= last;
        long long rowoff = 0;
        float sc = -FLT_MAX;
        bool counted = false;
        if (live) {
          const int page = checked_page(table[j / page_size], num_pages, status);
          if (page >= 0) {  // else: an id beyond the pool (the status flag is set); the key counts for nothing
            rowoff = (((long long)page * nkv + kvh) * page_size + (j % page_size)) * ROW;
            sc = dot_key<T>(cache + rowoff + koff, qs[warp]) * hscale;
            if (softcap > 0.f) sc = softcap * tanhf(sc * inv_cap);
            sc += hbias;
            counted = true;
          }
        }
        float pj;
        if constexpr (SIGMOID) {
          pj = counted ? 1.f / (1.f + expf(-sc)) : 0.f;
        } else {
          const float bm = warp_max(sc);
          const float m_new = fmaxf(m, bm);
          const float alpha = expf(m - m_new);
          pj = counted ? expf(sc - m_new) : 0.f;
          l = l * alpha + warp_sum(pj);
          m = m_new;
#pragma unroll
          for (int i = 0; i < DPL; i++) acc[i] *= alpha;
        }
        const int nlive = (last - base + 1) < 32 ? (last - base + 1) : 32;
        for (int jj = 0; jj < nlive; jj++) {
          const float pv = __shfl_sync(0xffffffffu, pj, jj);
          const long long ro = __shfl_sync(0xffffffffu, rowoff, jj);
          const T* vrow = cache + ro + KW;
#pragma unroll
          for (int i = 0; i < DPL; i++) {
            const int d = lane + 32 * i;
            if (d < VD) acc[i] = fmaf(pv, to_float(vrow[d]), acc[i]);
          }
        }
      }
    }
    const float inv_l = SIGMOID ? 1.f : (l > 0.f ? 1.f / l : 0.f);
    TO* orow = out + ((size_t)blockIdx.x * nh * MAPS + h) * VD;
#pragma unroll
    for (int i = 0; i < DPL; i++) {
      const int d = lane + 32 * i;
      if (d < VD) orow[d] = from_float<TO>(acc[i] * inv_l);
    }
    __syncwarp();
  }
}

// The differential form's combination (two maps): a float32 [rows, heads, 2, VD];
//   o = a_0 - lambda a_1,   out = o / sqrt(mean(o^2) + eps) * mult * sigmoid(gate[token][head])
// gate: float32, row stride gate_stride, the heads' logits from column gate_off on (null: no gate); rows names the
// tokens the rows of a belong to (null: row r is token r).  One warp a (row, head).
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
diff_combine_kernel(const float* __restrict__ a, const float* __restrict__ lambda, float eps, float mult,
                    const float* __restrict__ gate, int gate_stride, int gate_off, const int* __restrict__ rows,
                    T* __restrict__ out, int nh) {
  trigger_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x, lane = threadIdx.x & 31;
  const float lam = lambda[0];
  for (int h = threadIdx.x >> 5; h < nh; h += WARPS) {
    const float* a0 = a + ((size_t)r * nh + h) * MAPS * VD;
    float o[DPL], ss = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; i++) {
      const int d = lane + 32 * i;
      o[i] = d < VD ? a0[d] - lam * a0[(MAPS > 1 ? VD : 0) + d] : 0.f;
      ss = fmaf(o[i], o[i], ss);
    }
    ss = warp_sum(ss);
    float f = rsqrtf(ss / (float)VD + eps) * mult;
    if (gate != nullptr) f *= 1.f / (1.f + expf(-gate[(size_t)(rows ? rows[r] : r) * gate_stride + gate_off + h]));
#pragma unroll
    for (int i = 0; i < DPL; i++) {
      const int d = lane + 32 * i;
      if (d < VD) out[((size_t)r * nh + h) * VD + d] = from_float<T>(o[i] * f);
    }
  }
}

template <typename T>
int prep_launch(const float* qkv, int stride, const float* bias, int unit_norm, float eps, void* q_out, void* cache,
                const int* positions, const int* token_seq, const int* page_indptr, const int* page_ids, int n_tokens,
                int nh, int nkv, int page_size, int num_pages, int write_cache, int* status, const float* norm_w,
                const double* freq, int rot_dims, int rot_pairs, int values_are_keys, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv != 0 || page_size <= 0) return -2;
  if (freq != nullptr && (rot_dims < 0 || rot_dims > QK || (rot_dims & 1))) return -2;
  if (values_are_keys && (QK != VD || MAPS != 1)) return -2;
  return launch_pdl(sink_attn_prep_kernel<T>, dim3(n_tokens), dim3(256), 0, st, qkv, stride, bias, unit_norm, eps,
                    (T*)q_out, (T*)cache, positions, token_seq, page_indptr, page_ids, nh, nkv, page_size, num_pages,
                    write_cache, status, norm_w, freq, rot_dims, rot_pairs, values_are_keys);
}

template <typename T>
int attn_launch(const void* q, void* out, const void* cache, const int* token_seq, const int* positions,
                const int* page_indptr, const int* page_ids, const int* rows, int n_rows, const float* sinks, int nh,
                int nkv, int page_size, float scale, float softcap, int window, int keep_first, int num_pages,
                int* status, const float* head_scale, const float* head_bias, cudaStream_t st) {
  if (n_rows <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || page_size <= 0 || keep_first < 0) return -2;
  if (nkv > 65535) return -3;
  return launch_pdl(attn_sink_simt_kernel<T>, dim3(n_rows, nkv), dim3(WARPS * 32), 0, st, (const T*)q,
                    (typename OutOf<T>::type*)out, (const T*)cache, token_seq, positions, page_indptr, page_ids, rows,
                    sinks, nh, nkv, page_size, scale, softcap, window, keep_first, num_pages, status, head_scale,
                    head_bias);
}

}  // namespace

#define TKB_SINK_EXPORTS(SUF, T)                                                                                      \
  TKB_EXPORT int tkb_sink_attn_prep_##SUF(const float* qkv, int stride, const float* bias, int unit_norm, float eps,  \
                                          void* q_out, void* cache, const int* positions, const int* token_seq,       \
                                          const int* page_indptr, const int* page_ids, int n_tokens, int nh, int nkv, \
                                          int page_size, int num_pages, int write_cache, int* status,                 \
                                          const float* norm_w, const double* freq, int rot_dims, int rot_pairs,       \
                                          int values_are_keys, void* st) {                                            \
    return prep_launch<T>(qkv, stride, bias, unit_norm, eps, q_out, cache, positions, token_seq, page_indptr,         \
                          page_ids, n_tokens, nh, nkv, page_size, num_pages, write_cache, status, norm_w, freq,       \
                          rot_dims, rot_pairs, values_are_keys, (cudaStream_t)st);                                    \
  }                                                                                                                   \
  TKB_EXPORT int tkb_attn_sink_simt_##SUF(const void* q, void* out, const void* cache, const int* token_seq,          \
                                          const int* positions, const int* page_indptr, const int* page_ids,          \
                                          const int* rows, int n_rows, const float* sinks, int nh, int nkv,           \
                                          int page_size, float scale, float softcap, int window, int keep_first,      \
                                          int num_pages, int* status, const float* head_scale,                        \
                                          const float* head_bias, void* st) {                                         \
    return attn_launch<T>(q, out, cache, token_seq, positions, page_indptr, page_ids, rows, n_rows, sinks, nh, nkv,   \
                          page_size, scale, softcap, window, keep_first, num_pages, status, head_scale, head_bias,    \
                          (cudaStream_t)st);                                                                          \
  }                                                                                                                   \
  TKB_EXPORT int tkb_diff_combine_##SUF(const float* a, const float* lambda, float eps, float mult,                   \
                                        const float* gate, int gate_stride, int gate_off, const int* rows, void* out, \
                                        int n_rows, int nh, void* st) {                                               \
    if (n_rows <= 0) return 0;                                                                                        \
    if (MAPS != 2 || nh <= 0) return -2;                                                                              \
    return launch_pdl(diff_combine_kernel<T>, dim3(n_rows), dim3(WARPS * 32), 0, (cudaStream_t)st, a, lambda, eps,    \
                      mult, gate, gate_stride, gate_off, rows, (T*)out, nh);                                          \
  }

TKB_SINK_EXPORTS(f32, float)
TKB_SINK_EXPORTS(bf16, __nv_bfloat16)

// ------------------------------------------------------------------------------------------------ tensor cores
#if (TKB_QK % 16 == 0) && (TKB_VD % 16 == 0) && (TKB_QK <= 256) && (TKB_VD <= 256) && (TKB_MAPS != 3)
#define TKB_SINK_TC 1
namespace {

using bf16 = __nv_bfloat16;
constexpr int KT = 64;            // keys per staged tile
constexpr int RS = ROW + 8;       // row stride in shared memory (elements): 16 bytes of padding keep the banks apart
constexpr int KSTEPS = QK / 16;   // k-steps of q . k
constexpr int VT = VD / 8;        // 8-column tiles of the output
constexpr float NEG_BIG = -1e30f;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// cap * tanh(scale * d / cap) in units of log2 from the raw dot product d: tanh(x) = 1 - 2 / (e^(2x) + 1), five
// instructions a score.  k1 = 2 log2(e) scale / cap, so that e^(2x) = 2^(k1 d); an exponential that overflows gives
// tanh = 1, one that underflows tanh = -1, as they should.  The exponential and the reciprocal are each good to about
// 1e-7 of a result near 1, so the capped score is off by about cap * 1e-7: the size of a float32 rounding of a score of
// the cap's own size (the FP32-pipe kernel calls tanhf).  Without a cap: d * scale * log2(e).
// A number added to the score (a head's bias) enters as b2 = bias log2(e).
struct ScoreMap {
  float k1, c0, c1;  // capped: fma(rcp(ex2(k1 d) + 1), c1, c0) with c0 = cap log2(e) + b2, c1 = -2 cap log2(e);  plain: d * k1 + c0
  bool capped;
};
__device__ __forceinline__ ScoreMap score_map(float scale, float softcap, float bias = 0.f) {
  ScoreMap m;
  m.capped = softcap > 0.f;
  m.k1 = m.capped ? 2.f * LOG2E * scale / softcap : scale * LOG2E;
  m.c0 = (m.capped ? softcap * LOG2E : 0.f) + bias * LOG2E;
  m.c1 = -2.f * softcap * LOG2E;
  return m;
}
__device__ __forceinline__ float mapped_score(float d, const ScoreMap& m) {
  if (!m.capped) return fmaf(d, m.k1, m.c0);
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(ex2(d * m.k1) + 1.f));
  return fmaf(r, m.c1, m.c0);
}
// sigmoid of a score given in units of log2: 1 / (1 + 2^(-x)); an exponential that overflows gives 0
__device__ __forceinline__ float sigmoid2(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(ex2(-x) + 1.f));
  return r;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// Keys k0 .. k0 + 63 of the request into one buffer: a cached row [k | v] is one run of 16-byte pieces.  Rows outside
// [k_lo, k_hi], on a page that is gone or beyond the pool, are zeros.
__device__ __forceinline__ void stage_tile(bf16* buf, const bf16* __restrict__ cache, const int* __restrict__ table,
                                           int k0, int k_lo, int k_hi, int kvh, int nkv, int ps, int num_pages,
                                           bool& bad, int tid) {
  constexpr int CH = ROW / 8;
  for (int idx = tid; idx < KT * CH; idx += 128) {
    const int r = idx / CH, c = idx - r * CH;
    const int key = k0 + r;
    bf16* dst = buf + r * RS + c * 8;
    int page = -1;
    if (key >= k_lo && key <= k_hi) page = checked_page(table[key / ps], num_pages, bad);
    if (page >= 0) cp_async16(smem_u32(dst), cache + (((size_t)page * nkv + kvh) * ps + (key % ps)) * ROW + c * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// One warp, 16 rows, NT groups of 8 keys that start at row `kr0` of the staged tile (key index key0): scores, running
// softmax, and the weighted sum of values.  lim_lo / lim_hi: the keys each of the thread's two rows may see; keys
// below `keep` are seen from below lim_lo too (the first positions that a window keeps).  koff: where the map's key
// starts in a staged row.
// MASKED false: every key of the span is seen by every row (the caller has checked), no limit is looked at.
template <int NT, bool MASKED>
__device__ __forceinline__ void attend(const bf16* buf, int kr0, int key0, const uint32_t (&qf)[KSTEPS][4], float (&o)[VT][4],
                                       float (&m)[2], float (&l)[2], const int (&lim_lo)[2], const int (&lim_hi)[2],
                                       const ScoreMap (&sm)[2], int lane, int koff = 0, int keep = 0) {
  const int g = lane >> 2, t = lane & 3;
  float sc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++) {
    sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
    if constexpr (KSTEPS % 2 == 0) {
      // four 8 x 8 pieces a load: keys nt * 8 .. + 7, key channels of two k-steps (a piece's row is one key's 8 channels)
      const bf16* kp = buf + (kr0 + nt * 8 + (lane & 7)) * RS + koff + (lane >> 3) * 8;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ks += 2) {
        uint32_t b[4];
        ldmatrix_x4(b, smem_u32(kp + ks * 16));
        mma_bf16(sc[nt], qf[ks], b[0], b[1]);
        mma_bf16(sc[nt], qf[ks + 1], b[2], b[3]);
      }
    } else {
      const bf16* krow = buf + (kr0 + nt * 8 + g) * RS + koff + 2 * t;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ks++) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + ks * 16);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + ks * 16 + 8);
        mma_bf16(sc[nt], qf[ks], b0, b1);
      }
    }
  }
  if constexpr (SIGMOID) {
    // no softmax: a key's weight is the sigmoid of its score, keys out of sight weigh nothing; m and l stay as they are
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          float v = sigmoid2(mapped_score(sc[nt][h * 2 + e], sm[h]));
          if (MASKED) {
            const int key = key0 + nt * 8 + 2 * t + e;
            if ((key < lim_lo[h] && key >= keep) || key > lim_hi[h]) v = 0.f;
          }
          sc[nt][h * 2 + e] = v;
        }
  } else {
  float alpha[2];
#pragma unroll
  for (int h = 0; h < 2; h++) {
    float mx = NEG_BIG;
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        float v = mapped_score(sc[nt][h * 2 + e], sm[h]);
        if (MASKED) {
          const int key = key0 + nt * 8 + 2 * t + e;
          if ((key < lim_lo[h] && key >= keep) || key > lim_hi[h]) v = -INFINITY;
        }
        sc[nt][h * 2 + e] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[h], mx);
    alpha[h] = ex2(m[h] - m_new);
    m[h] = m_new;
    float sum = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int e = 0; e < 2; e++) {
        const float p = ex2(sc[nt][h * 2 + e] - m_new);
        sc[nt][h * 2 + e] = p;
        sum += p;
      }
    l[h] = l[h] * alpha[h] + sum;  // this thread's share; the four threads of a row are added up at the end
  }
#pragma unroll
  for (int vt = 0; vt < VT; vt++) {
    o[vt][0] *= alpha[0];
    o[vt][1] *= alpha[0];
    o[vt][2] *= alpha[1];
    o[vt][3] *= alpha[1];
  }
  }
#pragma unroll
  for (int kk = 0; kk < NT / 2; kk++) {  // 16 keys at a time
    uint32_t pf[4] = {pack_bf16(sc[2 * kk][0], sc[2 * kk][1]), pack_bf16(sc[2 * kk][2], sc[2 * kk][3]),
                      pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]), pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3])};
    const bf16* vbase = buf + (kr0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * RS + KW + (lane >> 4) * 8;
#pragma unroll
    for (int vt = 0; vt < VT; vt += 2) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, smem_u32(vbase + vt * 8));
      mma_bf16(o[vt], pf, b[0], b[1]);
      mma_bf16(o[vt + 1], pf, b[2], b[3]);
    }
  }
}

constexpr size_t TC_SMEM = (size_t)2 * KT * RS * sizeof(bf16);

// Portions: blockIdx.y counts the 64-query tiles of the step's requests that bring more than one token from the end;
// blockIdx.x is the query head.
__global__ void __launch_bounds__(128)
attn_sink_tiles_kernel(const bf16* __restrict__ q, OutOf<bf16>::type* __restrict__ out, const bf16* __restrict__ cache,
                       const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                       const int* __restrict__ seq_kv_len, const int* __restrict__ page_indptr,
                       const int* __restrict__ page_ids, int n_seqs, const float* __restrict__ sinks, int nh, int nkv,
                       int ps, float scale, float softcap, int window, int keep_first, int num_pages, int* __restrict__ status,
                       const float* __restrict__ head_scale, const float* __restrict__ head_bias) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* bufs = reinterpret_cast<bf16*>(smem_raw);
  trigger_dependents();
  // the last tiles first, for all heads: without a window a portion's last queries see the most keys, and the blocks
  // that start first should be the ones that run longest (blocks start in the order of blockIdx.x, then blockIdx.y)
  int s = 0, tile = (int)gridDim.y - 1 - (int)blockIdx.y;
  for (; s < n_seqs; s++) {
    const int n = seq_q_len[s];
    const int tiles = n > 1 ? (n + KT - 1) / KT : 0;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (s >= n_seqs) return;
  grid_dependency_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  // blockIdx.x counts (head, map) as query heads
  const int h = blockIdx.x, kvh = (h / MAPS) / (nh / nkv), koff = (h % MAPS) * QK, nhm = nh * MAPS;
  const int n_q = seq_q_len[s], start = seq_q_start[s];
  const int pos0 = seq_kv_len[s] - n_q;  // position of the portion's first token
  const int r0 = tile * KT;              // first query of the tile within the portion
  const int rows = min(KT, n_q - r0);
  const int* table = page_ids + page_indptr[s];
  const ScoreMap sm1 = score_map(scale * (head_scale ? head_scale[h] : 1.f), softcap, head_bias ? head_bias[h] : 0.f);
  const ScoreMap sm[2] = {sm1, sm1};

  uint32_t qf[KSTEPS][4];
  int lim_lo[2], lim_hi[2];
#pragma unroll
  for (int hh = 0; hh < 2; hh++) {
    const int r = warp * 16 + g + hh * 8;
    const bool live = r < rows;
    const int p = pos0 + r0 + r;
    lim_hi[hh] = live ? p : -1;
    lim_lo[hh] = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const bf16* qrow = q + ((size_t)(start + r0 + (live ? r : 0)) * nhm + h) * QK;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) {
      qf[ks][hh] = live ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t) : 0u;
      qf[ks][hh + 2] = live ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t) : 0u;
    }
  }
  // (the sigmoid form never touches m and l: a sum of 1 makes the division at the end the identity)
  const float sink2 = SIGMOID ? 0.f : (sinks ? sinks[h] * LOG2E : NEG_BIG);
  const bool open = SIGMOID || sinks != nullptr;
  float m[2] = {sink2, sink2};
  float l[2] = {(open && t == 0) ? 1.f : 0.f, (open && t == 0) ? 1.f : 0.f};
  float o[VT][4];
#pragma unroll
  for (int vt = 0; vt < VT; vt++) o[vt][0] = o[vt][1] = o[vt][2] = o[vt][3] = 0.f;

  const int p_first = pos0 + r0, p_last = pos0 + r0 + rows - 1;
  const int k_lo = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
  // the first positions that the window keeps in sight: [0, kept) lies before every row's window and is staged in
  // tiles of its own, which come first; kept positions from k_lo on arrive with the window's tiles
  const int keep = window > 0 ? keep_first : 0;
  const int kept = min(keep, k_lo);
  const int keep_tiles = (kept + KT - 1) / KT;
  const int n_tiles = keep_tiles + (p_last - k_lo) / KT + 1;
  auto tile_key0 = [&](int it) { return it < keep_tiles ? it * KT : k_lo + (it - keep_tiles) * KT; };
  auto tile_first = [&](int it) { return it < keep_tiles ? 0 : k_lo; };
  auto tile_last = [&](int it) { return it < keep_tiles ? kept - 1 : p_last; };
  // the keys this warp's rows can see within the window's tiles: [w_lo, w_hi]
  const int w_first = pos0 + r0 + warp * 16;
  const int w_lo = keep > k_lo ? k_lo : ((window > 0 && w_first - window + 1 > 0) ? w_first - window + 1 : 0);
  const int w_hi = min(p_last, w_first + 15);
  const int w_last_lo = (window > 0 && w_first + 15 - window + 1 > 0) ? w_first + 15 - window + 1 : 0;  // the last row's
  bool bad = false;
  stage_tile(bufs, cache, table, tile_key0(0), tile_first(0), tile_last(0), kvh, nkv, ps, num_pages, bad, tid);
  cp_async_commit();
  for (int it = 0; it < n_tiles; it++) {
    bf16* cur = bufs + (it & 1) * KT * RS;
    if (it + 1 < n_tiles) {
      stage_tile(bufs + ((it + 1) & 1) * KT * RS, cache, table, tile_key0(it + 1), tile_first(it + 1), tile_last(it + 1), kvh,
                 nkv, ps, num_pages, bad, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = tile_key0(it);
    if (it < keep_tiles) {
      // kept positions: every live row sees [0, kept), nothing beyond in this tile
      if (warp * 16 < rows) {
        const int kl[2] = {0, 0}, kh[2] = {lim_hi[0] < 0 ? -1 : kept - 1, lim_hi[1] < 0 ? -1 : kept - 1};
        attend<8, true>(cur, 0, key0, qf, o, m, l, kl, kh, sm, lane, koff, 0);
      }
    } else if (warp * 16 < rows && key0 <= w_hi && key0 + KT - 1 >= w_lo) {  // warp-uniform: some row of the warp sees some key
      // all 16 rows live and the whole tile inside every row's window and before the warp's first query: no masks
      if (warp * 16 + 16 <= rows && key0 + KT - 1 <= w_first && key0 >= w_last_lo)
        attend<8, false>(cur, 0, key0, qf, o, m, l, lim_lo, lim_hi, sm, lane, koff, keep);
      else
        attend<8, true>(cur, 0, key0, qf, o, m, l, lim_lo, lim_hi, sm, lane, koff, keep);
    }
    __syncthreads();  // the buffer is free for the tile after next
  }
  report_bad_page(bad, status);
#pragma unroll
  for (int hh = 0; hh < 2; hh++) {
    l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 1);
    l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 2);
    const int r = warp * 16 + g + hh * 8;
    if (r < rows) {
      const float inv = l[hh] > 0.f ? 1.f / l[hh] : 0.f;
      auto* orow = out + ((size_t)(start + r0 + r) * nhm + h) * VD + 2 * t;
#pragma unroll
      for (int vt = 0; vt < VT; vt++) {
        if constexpr (MAPS > 1)
          *reinterpret_cast<float2*>(orow + vt * 8) = make_float2(o[vt][hh * 2] * inv, o[vt][hh * 2 + 1] * inv);
        else
          *reinterpret_cast<uint32_t*>(orow + vt * 8) = pack_bf16(o[vt][hh * 2] * inv, o[vt][hh * 2 + 1] * inv);
      }
    }
  }
}

// Single tokens: blockIdx.x = request row (it leaves unless the request brings one token), blockIdx.y = key/value
// head * head tiles + head tile (16 query heads a tile).  With several maps a head the block's four warps are shared
// out among the maps (all maps read the tile that the block stages once), and a map's warps share out a tile's keys.
constexpr int WPM = 4 / MAPS;   // warps a map
constexpr int KPW = KT / WPM;   // keys of a tile a warp takes
__global__ void __launch_bounds__(128)
attn_sink_single_kernel(const bf16* __restrict__ q, OutOf<bf16>::type* __restrict__ out, const bf16* __restrict__ cache,
                        const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                        const int* __restrict__ seq_kv_len, const int* __restrict__ page_indptr,
                        const int* __restrict__ page_ids, const float* __restrict__ sinks, int nh, int nkv, int head_tiles,
                        int ps, float scale, float softcap, int window, int keep_first, int num_pages,
                        int* __restrict__ status, float* __restrict__ part, const float* __restrict__ head_scale,
                        const float* __restrict__ head_bias) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* bufs = reinterpret_cast<bf16*>(smem_raw);
  trigger_dependents();
  const int s = blockIdx.x;
  if (seq_q_len[s] != 1) return;
  const int splits = gridDim.z, split = blockIdx.z;
  grid_dependency_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int group = nh / nkv;
  const int kvh = blockIdx.y / head_tiles, g0 = (blockIdx.y - kvh * head_tiles) * 16;
  const int map = warp / WPM, wsub = warp % WPM, koff = map * QK, nhm = nh * MAPS;
  const int gn = min(16, group - g0);
  const int tok = seq_q_start[s];
  const int p = seq_kv_len[s] - 1;
  const int* table = page_ids + page_indptr[s];
  ScoreMap sm[2];
  const int k_lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;

  uint32_t qf[KSTEPS][4];
  float m[2], l[2];
#pragma unroll
  for (int hh = 0; hh < 2; hh++) {
    const int r = g + hh * 8;
    const bool live = r < gn;
    const int head = (kvh * group + g0 + (live ? r : 0)) * MAPS + map;  // (head, map) counted as a query head
    const bf16* qrow = q + ((size_t)tok * nhm + head) * QK;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) {
      qf[ks][hh] = live ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t) : 0u;
      qf[ks][hh + 2] = live ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t) : 0u;
    }
    sm[hh] = score_map(scale * (head_scale ? head_scale[head] : 1.f), softcap, head_bias ? head_bias[head] : 0.f);
    // (the sigmoid form: every share has maximum 0, and ONE share carries the sum 1, so the merges below only add)
    m[hh] = SIGMOID ? 0.f : (sinks ? sinks[head] * LOG2E : NEG_BIG);
    l[hh] = ((SIGMOID || sinks) && split == 0 && wsub == 0 && t == 0) ? 1.f : 0.f;  // the sink counts once: in one warp's sums
  }
  float o[VT][4];
#pragma unroll
  for (int vt = 0; vt < VT; vt++) o[vt][0] = o[vt][1] = o[vt][2] = o[vt][3] = 0.f;

  // the request's tiles are shared out evenly among the splits (blockIdx.z); a split may be left without any.  The
  // first positions that the window keeps in sight, [0, kept), have tiles of their own, which come first.
  const int kept = window > 0 ? min(keep_first, k_lo) : 0;
  const int keep_tiles = (kept + KT - 1) / KT;
  const int all_tiles = keep_tiles + (p - k_lo) / KT + 1;
  const int per_split = (all_tiles + splits - 1) / splits;
  const int it0 = split * per_split;
  const int n_tiles = min(all_tiles, it0 + per_split) - it0;
  auto tile_key0 = [&](int it) { return it < keep_tiles ? it * KT : k_lo + (it - keep_tiles) * KT; };
  auto tile_first = [&](int it) { return it < keep_tiles ? 0 : k_lo; };
  auto tile_last = [&](int it) { return it < keep_tiles ? kept - 1 : p; };
  bool bad = false;
  if (n_tiles > 0)
    stage_tile(bufs, cache, table, tile_key0(it0), tile_first(it0), tile_last(it0), kvh, nkv, ps, num_pages, bad, tid);
  cp_async_commit();
  for (int it = 0; it < n_tiles; it++) {
    bf16* cur = bufs + (it & 1) * KT * RS;
    if (it + 1 < n_tiles) {
      stage_tile(bufs + ((it + 1) & 1) * KT * RS, cache, table, tile_key0(it0 + it + 1), tile_first(it0 + it + 1),
                 tile_last(it0 + it + 1), kvh, nkv, ps, num_pages, bad, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = tile_key0(it0 + it) + wsub * KPW;
    const int last = tile_last(it0 + it);
    if (key0 <= last) {
      const int tl[2] = {tile_first(it0 + it), tile_first(it0 + it)}, th[2] = {last, last};
      attend<KPW / 8, true>(cur, wsub * KPW, key0, qf, o, m, l, tl, th, sm, lane, koff, 0);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  report_bad_page(bad, status);
#pragma unroll
  for (int hh = 0; hh < 2; hh++) {
    l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 1);
    l[hh] += __shfl_xor_sync(0xffffffffu, l[hh], 2);
  }
  // the four warps' partial results through shared memory (the tile buffers are free now)
  constexpr int SO = VD + 8;
  static_assert((size_t)(4 * 16 * SO + 4 * 16 * 2) * sizeof(float) <= TC_SMEM, "the merge scratch fits the tile buffers");
  float* so = reinterpret_cast<float*>(smem_raw);
  float* sml = so + 4 * 16 * SO;
#pragma unroll
  for (int vt = 0; vt < VT; vt++) {
    float* b = so + (warp * 16 + g) * SO + vt * 8 + 2 * t;
    *reinterpret_cast<float2*>(b) = make_float2(o[vt][0], o[vt][1]);
    *reinterpret_cast<float2*>(b + 8 * SO) = make_float2(o[vt][2], o[vt][3]);
  }
  if (t == 0) {
    sml[(warp * 16 + g) * 2] = m[0];
    sml[(warp * 16 + g) * 2 + 1] = l[0];
    sml[(warp * 16 + g + 8) * 2] = m[1];
    sml[(warp * 16 + g + 8) * 2 + 1] = l[1];
  }
  __syncthreads();
  for (int idx = tid; idx < MAPS * gn * VD; idx += 128) {
    const int mp = idx / (gn * VD), r = (idx - mp * gn * VD) / VD, d = idx - (mp * gn + r) * VD;
    float mm = NEG_BIG;
#pragma unroll
    for (int w = mp * WPM; w < (mp + 1) * WPM; w++) mm = fmaxf(mm, sml[(w * 16 + r) * 2]);
    float acc = 0.f, ll = 0.f;
#pragma unroll
    for (int w = mp * WPM; w < (mp + 1) * WPM; w++) {
      const float f = exp2f(sml[(w * 16 + r) * 2] - mm);
      acc += f * so[(w * 16 + r) * SO + d];
      ll += f * sml[(w * 16 + r) * 2 + 1];
    }
    const int head = (kvh * group + g0 + r) * MAPS + mp;
    if (splits == 1) {
      out[((size_t)tok * nhm + head) * VD + d] = from_float<OutOf<bf16>::type>(ll > 0.f ? acc / ll : 0.f);
    } else {  // this split's share: sums relative to its own maximum, for attn_sink_merge
      float* pr = part + (((size_t)s * nhm + head) * splits + split) * (VD + 2);
      pr[d] = acc;
      if (d == 0) {
        pr[VD] = mm;
        pr[VD + 1] = ll;
      }
    }
  }
}

// The splits of every single-token request put together: grid (request row, query head).
__global__ void attn_sink_merge_kernel(const float* __restrict__ part, OutOf<bf16>::type* __restrict__ out,
                                       const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len, int nh,
                                       int splits) {
  trigger_dependents();
  grid_dependency_wait();
  const int s = blockIdx.x, head = blockIdx.y;
  if (seq_q_len[s] != 1) return;
  const float* pr = part + ((size_t)s * nh + head) * splits * (VD + 2);
  float mm = NEG_BIG;
  for (int z = 0; z < splits; z++) mm = fmaxf(mm, pr[z * (VD + 2) + VD]);
  float ll = 0.f;
  for (int z = 0; z < splits; z++) ll += exp2f(pr[z * (VD + 2) + VD] - mm) * pr[z * (VD + 2) + VD + 1];
  const float inv = ll > 0.f ? 1.f / ll : 0.f;
  for (int d = threadIdx.x; d < VD; d += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < splits; z++) acc += exp2f(pr[z * (VD + 2) + VD] - mm) * pr[z * (VD + 2) + d];
    out[((size_t)seq_q_start[s] * nh + head) * VD + d] = from_float<OutOf<bf16>::type>(acc * inv);
  }
}

}  // namespace

// Attention of every token of the step (bfloat16): requests with one token through attn_sink_single, longer portions
// through attn_sink_tiles.  n_tokens and n_seqs size the grids; the blocks read the rest from the request table.
// splits > 1: a single-token request's tiles are shared out among so many blocks, whose shares meet in `part`
// (float32 [n_seqs * nh * splits * (VD + 2)]) and are put together by attn_sink_merge.
TKB_EXPORT int tkb_attn_sink_tc_bf16(const void* q, void* out, const void* cache, const int* seq_q_start,
                                     const int* seq_q_len, const int* seq_kv_len, const int* page_indptr,
                                     const int* page_ids, int n_tokens, int n_seqs, int portions, int singles,
                                     const float* sinks, int nh, int nkv, int page_size, float scale, float softcap,
                                     int window, int keep_first, int num_pages, int* status, float* part, int splits,
                                     const float* head_scale, const float* head_bias, void* st) {
  using TO = OutOf<bf16>::type;
  if (n_tokens <= 0 || n_seqs <= 0) return 0;
  if (nkv <= 0 || nh % nkv != 0 || page_size <= 0 || keep_first < 0) return -2;
  const int head_tiles = (nh / nkv + 15) / 16;
  if (nh * MAPS > 65535 || nkv * head_tiles > 65535) return -3;
  if (TC_SMEM > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attn_sink_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_sink_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM);
    if (e != cudaSuccess) return (int)e;
  }
  int rc = 0;
  if (splits < 1 || part == nullptr) splits = 1;
  if (splits > 64) return -2;
  if (singles) {
    rc = launch_pdl(attn_sink_single_kernel, dim3(n_seqs, nkv * head_tiles, splits), dim3(128), TC_SMEM,
                    (cudaStream_t)st, (const bf16*)q, (TO*)out, (const bf16*)cache, seq_q_start, seq_q_len, seq_kv_len,
                    page_indptr, page_ids, sinks, nh, nkv, head_tiles, page_size, scale, softcap, window, keep_first,
                    num_pages, status, part, head_scale, head_bias);
    if (rc == 0 && splits > 1)
      rc = launch_pdl(attn_sink_merge_kernel, dim3(n_seqs, nh * MAPS), dim3(VD >= 128 ? 128 : 64), 0, (cudaStream_t)st,
                      (const float*)part, (TO*)out, seq_q_start, seq_q_len, nh * MAPS, splits);
  }
  if (rc != 0 || !portions) return rc;
  const int tiles = n_tokens / KT + n_seqs;  // no step of this shape has more 64-query tiles
  if (tiles > 65535) return -3;
  return launch_pdl(attn_sink_tiles_kernel, dim3(nh * MAPS, tiles), dim3(128), TC_SMEM, (cudaStream_t)st, (const bf16*)q,
                    (TO*)out, (const bf16*)cache, seq_q_start, seq_q_len, seq_kv_len, page_indptr, page_ids, n_seqs,
                    sinks, nh, nkv, page_size, scale, softcap, window, keep_first, num_pages, status, head_scale,
                    head_bias);
}
#endif  // tensor-core sizes
TKB_EXPORT int tkb_attn_sink_has_tc() {
#ifdef TKB_SINK_TC
  return 1;
#else
  return 0;
#endif
}
