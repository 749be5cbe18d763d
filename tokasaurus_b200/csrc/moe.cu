// Routed experts (mixture of experts): the router with its choice of the `top` largest logits and the softmax over
// the chosen ones (float32), the ordering of a step's (token, choice) pairs by expert, the experts' products over
// that ordering (each block finds its expert from the offsets on the device, so nothing is read back to the host),
// and the weighted sum of the chosen experts' outputs.  Built for float and bfloat16 activations.
//
// A second way of choosing (moe_choose_scored): scores s = sigmoid(logits); the choice goes by s + correction (a
// learned vector that takes no part in the weights), among the experts of the best `keep` of `groups` equal groups of
// neighbours only (a group scores the sum of its two largest choice scores); the weights are the chosen experts' s over
// their sum (+ 1e-20), times a scale.  A second kind of expert: down(gelu(up h)) with the exact (erf) GELU, no gate.
#include "common.cuh"
#include <float.h>

using namespace tkb;

namespace {

// ------------------------------------------------------------------------------------------------
// Router, first kernel: logits z[t][e] = h[t] . Wr[e] + b[e] in float32 (Wr float32 [E, H]).  Block (x, y): four
// tokens (one a warp) times four experts; the token's row is read once for the four experts, four sums run side by
// side, and the four warps of a block read the same weight rows (one trip to the L2 for the four).  Few tokens
// (decoding) still make tokens x E / 4 warps.
constexpr int ROUTE_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_logits_kernel(const T* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ br,
                  float* __restrict__ z, int n_tokens, int H, int E) {
  trigger_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  const int e0 = blockIdx.y * 4;
  if (t >= n_tokens) return;
  const T* hr = h + (size_t)t * H;
  const float* w0 = wr + (size_t)e0 * H;
  const float* w1 = wr + (size_t)min(e0 + 1, E - 1) * H;
  const float* w2 = wr + (size_t)min(e0 + 2, E - 1) * H;
  const float* w3 = wr + (size_t)min(e0 + 3, E - 1) * H;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  if ((H & 3) == 0 && (((uintptr_t)wr) & 15) == 0) {
    // sixteen bytes of every weight row a lane and pass; the loads of four passes are issued before their sums (with
    // two in flight, eight tokens of width 2,048 waited eight times for memory: 18 us a layer); passes beyond the row
    // add zeros, and the sums keep their order
    for (int i0 = lane * 4; i0 < H; i0 += 512) {
      float4 v[4][4];
      float x[4][4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const int i = i0 + 128 * u;
        const bool in = i < H;
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        v[u][0] = in ? *reinterpret_cast<const float4*>(w0 + i) : zero;
        v[u][1] = in ? *reinterpret_cast<const float4*>(w1 + i) : zero;
        v[u][2] = in ? *reinterpret_cast<const float4*>(w2 + i) : zero;
        v[u][3] = in ? *reinterpret_cast<const float4*>(w3 + i) : zero;
#pragma unroll
        for (int c = 0; c < 4; c++) x[u][c] = in ? to_float(hr[i + c]) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        a0 = fmaf(x[u][0], v[u][0].x, fmaf(x[u][1], v[u][0].y, fmaf(x[u][2], v[u][0].z, fmaf(x[u][3], v[u][0].w, a0))));
        a1 = fmaf(x[u][0], v[u][1].x, fmaf(x[u][1], v[u][1].y, fmaf(x[u][2], v[u][1].z, fmaf(x[u][3], v[u][1].w, a1))));
        a2 = fmaf(x[u][0], v[u][2].x, fmaf(x[u][1], v[u][2].y, fmaf(x[u][2], v[u][2].z, fmaf(x[u][3], v[u][2].w, a2))));
        a3 = fmaf(x[u][0], v[u][3].x, fmaf(x[u][1], v[u][3].y, fmaf(x[u][2], v[u][3].z, fmaf(x[u][3], v[u][3].w, a3))));
      }
    }
  } else {
#pragma unroll 4
    for (int i = lane; i < H; i += 32) {
      const float x = to_float(hr[i]);
      a0 = fmaf(x, w0[i], a0);
      a1 = fmaf(x, w1[i], a1);
      a2 = fmaf(x, w2[i], a2);
      a3 = fmaf(x, w3[i], a3);
    }
  }
  a0 = warp_sum(a0); a1 = warp_sum(a1); a2 = warp_sum(a2); a3 = warp_sum(a3);
  if (lane == 0) {
    const float acc[4] = {a0, a1, a2, a3};
    for (int u = 0; u < 4 && e0 + u < E; u++) z[(size_t)t * E + e0 + u] = acc[u] + (br != nullptr ? br[e0 + u] : 0.f);
  }
}

// Router, second kernel: one warp a token takes the `top` largest logits one after the other (equal logits: the
// lower expert first); weights = softmax over the chosen logits, or (over_all) the chosen experts' shares of the
// softmax over ALL experts, not renormalised; both times a number `scale`.  Rows of padding tokens choose nothing.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_choose_kernel(const float* __restrict__ z_all, const int* __restrict__ token_seq, int* __restrict__ top_idx,
                  float* __restrict__ top_w, int n_tokens, int E, int top, int over_all, float scale) {
  extern __shared__ float zs[];  // [warps][E]
  trigger_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= n_tokens) return;
  if (token_seq != nullptr && token_seq[t] < 0) {
    for (int k = lane; k < top; k += 32) {
      top_idx[(size_t)t * top + k] = -1;
      top_w[(size_t)t * top + k] = 0.f;
    }
    return;
  }
  float* z = zs + (size_t)warp * E;
  for (int e = lane; e < E; e += 32) z[e] = z_all[(size_t)t * E + e];
  __syncwarp();
  float first = 0.f, denom = 0.f, all = 0.f;
  if (over_all) {  // the sum of exp(z - max) over every expert, before the choice overwrites what it takes
    float mx = -FLT_MAX;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    for (int e = lane; e < E; e += 32) all += expf(z[e] - mx);
    all = warp_sum(all);
  }
  for (int k = 0; k < top; k++) {
    float best = -FLT_MAX;
    int arg = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best) { best = v; arg = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (k == 0) first = best;
    const float p = expf(best - first);
    denom += p;
    if (lane == 0) {
      top_idx[(size_t)t * top + k] = arg;
      top_w[(size_t)t * top + k] = p;
      if (arg < E) z[arg] = -FLT_MAX;
    }
    __syncwarp();
  }
  const float inv = scale / (over_all ? all : denom);
  __syncwarp();
  for (int k = lane; k < top; k += 32) top_w[(size_t)t * top + k] *= inv;
}

// Router, second kernel, the other way of choosing: one warp a token.  s = sigmoid(z), c = s + correction; group g holds
// experts g * per .. (g + 1) * per - 1 and scores the sum of its two largest c (its only c if per == 1); experts
// outside the `keep` best groups cannot be chosen (their c counts as minus infinity); the `top` largest c are chosen,
// equal scores: the lower expert (group) first; weights s / (sum of the chosen s + 1e-20) * scale.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_choose_scored_kernel(const float* __restrict__ z_all, const float* __restrict__ correction,
                         const int* __restrict__ token_seq, int* __restrict__ top_idx, float* __restrict__ top_w,
                         int n_tokens, int E, int top, int groups, int keep, float scale) {
  extern __shared__ float zs[];  // [warps][2 E + groups]: s, c, group scores
  trigger_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= n_tokens) return;
  if (token_seq != nullptr && token_seq[t] < 0) {
    for (int k = lane; k < top; k += 32) {
      top_idx[(size_t)t * top + k] = -1;
      top_w[(size_t)t * top + k] = 0.f;
    }
    return;
  }
  float* sv = zs + (size_t)warp * (2 * E + groups);
  float* cv = sv + E;
  float* gs = cv + E;
  for (int e = lane; e < E; e += 32) {
    const float s = 1.f / (1.f + expf(-z_all[(size_t)t * E + e]));
    sv[e] = s;
    cv[e] = s + (correction != nullptr ? correction[e] : 0.f);
  }
  __syncwarp();
  auto warp_argmax = [&](float& best, int& arg) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
  };
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float b1 = -FLT_MAX, b2 = -FLT_MAX;
      for (int e = g * per; e < (g + 1) * per; e++) {
        const float v = cv[e];
        if (v > b1) { b2 = b1; b1 = v; }
        else if (v > b2) b2 = v;
      }
      gs[g] = per > 1 ? b1 + b2 : b1;
    }
    __syncwarp();
    // take the `keep` best groups one after the other; a group that is taken gets the mark +inf
    for (int k = 0; k < keep; k++) {
      float best = -FLT_MAX;
      int arg = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && v > best) { best = v; arg = g; }
      }
      warp_argmax(best, arg);
      if (lane == 0 && arg < groups) gs[arg] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / per] != INFINITY) cv[e] = -INFINITY;
    __syncwarp();
  }
  float denom = 0.f;
  for (int k = 0; k < top; k++) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = cv[e];
      if (v > best) { best = v; arg = e; }
    }
    warp_argmax(best, arg);
    const float w = arg < E ? sv[arg] : 0.f;
    denom += w;
    __syncwarp();
    if (lane == 0) {
      top_idx[(size_t)t * top + k] = arg < E ? arg : -1;
      top_w[(size_t)t * top + k] = w;
      if (arg < E) cv[arg] = -INFINITY;
    }
    __syncwarp();
  }
  const float f = scale / (denom + 1e-20f);
  for (int k = lane; k < top; k += 32) top_w[(size_t)t * top + k] *= f;
}

// One block: offsets[e] .. is expert e's span of the ordering; order[p] is the (token, choice) pair at place p
// (token * top + choice), place_of[pair] its place (-1 for a padding token's pairs).  pad > 1: every span starts at
// a multiple of pad (the tensor-core product's row tile), offsets[e + 1] - offsets[e] is then the span with its
// padding; tile_group[i] (n_tiles entries) names the expert that owns row tile i of pad places, -1 for none; and
// src_token[p] (cap places) is the token whose row stands at place p, -1 at the padding.
__global__ void moe_order_kernel(const int* __restrict__ top_idx, int n_pairs, int E, int top, int pad,
                                 int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ place_of,
                                 int* __restrict__ tile_group, int n_tiles, int* __restrict__ src_token, int cap) {
  extern __shared__ int cnt[];  // [E] counts, then [E] cursors, then [E + 1] starts
  int* cursor = cnt + E;
  int* start = cursor + E;
  trigger_dependents();
  grid_dependency_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  if (src_token != nullptr)
    for (int p = threadIdx.x; p < cap; p += blockDim.x) src_token[p] = -1;
  __syncthreads();
  for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) {
    const int e = top_idx[a];
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; e++) {
      offsets[e] = run;
      cursor[e] = run;
      start[e] = run;
      run += (cnt[e] + pad - 1) / pad * pad;
    }
    offsets[E] = run;
    start[E] = run;
  }
  __syncthreads();
  if (tile_group != nullptr) {
    for (int i = threadIdx.x; i < n_tiles; i += blockDim.x) {
      int g = -1;
      for (int e = 0; e < E; e++)
        if (i * pad >= start[e] && i * pad < start[e] + cnt[e]) g = e;
      tile_group[i] = g;
    }
  }
  for (int a = threadIdx.x; a < n_pairs; a += blockDim.x) {
    const int e = top_idx[a];
    if (e >= 0 && e < E) {
      const int p = atomicAdd(&cursor[e], 1);
      order[p] = a;
      place_of[a] = p;
      if (src_token != nullptr && p < cap) src_token[p] = a / top;
    } else {
      place_of[a] = -1;
    }
  }
}

// dst[p] = src[src_token[p]] (zeros where src_token[p] < 0): the step's rows in the order of the experts' spans.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ src, const int* __restrict__ src_token, T* __restrict__ dst,
                                  int H) {
  trigger_dependents();
  grid_dependency_wait();
  const int p = blockIdx.x;
  const int t = src_token[p];
  T* d = dst + (size_t)p * H;
  if (t < 0) {
    for (int i = threadIdx.x; i < H; i += blockDim.x) d[i] = from_float<T>(0.f);
    return;
  }
  const T* r = src + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) d[i] = r[i];
}

// ------------------------------------------------------------------------------------------------
// The experts' products over the ordering, on the FP32 pipes with float32 sums (each output element is one
// sequential chain over K, whatever else is in the step):
//   plain:  C[p, n] = A[src(p), :] . W[e][n, :]                      (C float32 [places, N])
//   gated:  C[p, n] = silu(A[src(p), :] . W[e][n, :]) * (A[src(p), :] . W[e][N + n, :])      (W[e] is [2N, K])
//   gelu:   C[p, n] = gelu(A[src(p), :] . W[e][n, :]), the exact (erf) form, in A's type
// src(p) = order[p] / top if `order` is given (rows of the step's tokens), else p.  Block (x, y): column tile x of the
// y-th row tile, counted over the experts' spans in turn; blocks beyond the last tile leave at once.
constexpr int BM = 64, BN = 64, BK = 16;
constexpr int ACT_NONE = 0, ACT_GATED = 1, ACT_GELU = 2, ACT_CLAMPED = 3;
// the clamped gated unit: g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(alpha g) * (u + 1)
__device__ __forceinline__ float clamped_unit(float gate, float up, float limit, float alpha) {
  const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}
__device__ __forceinline__ float gelu_erf_f(float v) { return 0.5f * v * (1.f + erff(v * 0.70710678118654752f)); }

template <typename TA, typename TC, int ACT>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TA* __restrict__ A, int lda, const TA* __restrict__ W, TC* __restrict__ C, int ldc,
                const int* __restrict__ offsets, const int* __restrict__ order, int top, int E, int N, int K,
                float limit, float alpha) {
  constexpr bool GATED = ACT == ACT_GATED || ACT == ACT_CLAMPED;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[GATED ? BK : 1][BN + 4];
  __shared__ int src_row[BM];
  trigger_dependents();
  grid_dependency_wait();
  int tile = blockIdx.y, e = 0, p0 = 0, p1 = 0;
  for (; e < E; e++) {
    const int lo = offsets[e], hi = offsets[e + 1];
    const int tiles = (hi - lo + BM - 1) / BM;
    if (tile < tiles) {
      p0 = lo + tile * BM;
      p1 = hi;
      break;
    }
    tile -= tiles;
  }
  if (e >= E) return;
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * BN;
  if (tid < BM) {
    const int p = p0 + tid;
    src_row[tid] = p < p1 ? (order != nullptr ? order[p] / top : p) : -1;
  }
  __syncthreads();
  const TA* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
  const int tx = tid & 15, ty = tid >> 4;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4], acu[GATED ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) {
      acc[i][j] = 0.f;
      if (GATED) acu[i][j] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += BK) {
    const int sr = src_row[lrow];
    const int n = n0 + lrow;
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int k = k0 + lk + u;
      As[lk + u][lrow] = (sr >= 0 && k < K) ? to_float(A[(size_t)sr * lda + k]) : 0.f;
      Ws[lk + u][lrow] = (n < N && k < K) ? to_float(We[(size_t)n * K + k]) : 0.f;
      if (GATED) Us[lk + u][lrow] = (n < N && k < K) ? to_float(We[(size_t)(N + n) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[4], b[4], c[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        b[j] = Ws[kk][tx * 4 + j];
        if (GATED) c[j] = Us[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if (GATED) acu[i][j] = fmaf(a[i], c[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int p = p0 + ty * 4 + i;
    if (p >= p1) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (ACT == ACT_CLAMPED) v = clamped_unit(v, acu[i][j], limit, alpha);
      else if (GATED) v = v / (1.f + expf(-v)) * acu[i][j];
      if (ACT == ACT_GELU) v = gelu_erf_f(v);
      C[(size_t)p * ldc + n] = from_float<TC>(v);
    }
  }
}

// The same products for steps of few rows (decoding): what counts then is that every weight is fetched once and at
// full width.  Block (x, e) owns 32 output features of expert e and all rows of e's span (none: it leaves); a warp
// takes two features at a time and streams their weight rows with 16-byte loads, eight rows of the span a pass
// (their activations are small and stay in the L1 cache), float32 sums, one chain a (row, feature).  Measured
// against a form with four lanes a feature (fewer shuffles, weight rows fetched in 64-byte pieces): this one is
// 2.7 times faster at 16 pairs and 2.9 times at 128.
constexpr int GV_ROWS = 8, GV_WARPS = 8, GV_FEATS = 32;
constexpr int GEMV_PLACES_MAX = 512;  // (token, choice) pairs up to which this form is used

template <typename T> struct Vec8;  // eight consecutive values as floats
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};

template <typename TA, typename TC, int ACT>
__global__ void __launch_bounds__(GV_WARPS * 32)
moe_gemv_kernel(const TA* __restrict__ A, int lda, const TA* __restrict__ W, TC* __restrict__ C, int ldc,
                const int* __restrict__ offsets, const int* __restrict__ order, int top, int N, int K, float limit,
                float alpha) {
  constexpr bool GATED = ACT == ACT_GATED || ACT == ACT_CLAMPED;
  trigger_dependents();
  grid_dependency_wait();
  const int e = blockIdx.y;
  const int p_lo = offsets[e], p_hi = offsets[e + 1];
  if (p_hi <= p_lo) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const TA* We = W + (size_t)e * (GATED ? 2 : 1) * N * K;
  for (int r0 = p_lo; r0 < p_hi; r0 += GV_ROWS) {
    const int nr = min(GV_ROWS, p_hi - r0);
    const TA* arow[GV_ROWS];
#pragma unroll
    for (int r = 0; r < GV_ROWS; r++) {
      const int p = r0 + min(r, nr - 1);
      arow[r] = A + (size_t)(order != nullptr ? order[p] / top : p) * lda;
    }
    for (int f0 = blockIdx.x * GV_FEATS + warp * 2; f0 < min(N, (int)(blockIdx.x + 1) * GV_FEATS); f0 += GV_WARPS * 2) {
      const int f1 = min(f0 + 1, N - 1);
      const TA* wg0 = We + (size_t)f0 * K;
      const TA* wg1 = We + (size_t)f1 * K;
      float acc[2][GV_ROWS], acu[GATED ? 2 : 1][GV_ROWS];
#pragma unroll
      for (int r = 0; r < GV_ROWS; r++) {
        acc[0][r] = acc[1][r] = 0.f;
        acu[0][r] = 0.f;
        if (GATED) acu[1][r] = 0.f;
      }
      for (int k = lane * 8; k < K; k += 32 * 8) {
        float w0[8], w1[8], u0[8], u1[8];
        Vec8<TA>::load(wg0 + k, w0);
        Vec8<TA>::load(wg1 + k, w1);
        if (GATED) {
          Vec8<TA>::load(wg0 + (size_t)N * K + k, u0);
          Vec8<TA>::load(wg1 + (size_t)N * K + k, u1);
        }
#pragma unroll
        for (int r = 0; r < GV_ROWS; r++) {
          if (r < nr) {
            float a[8];
            Vec8<TA>::load(arow[r] + k, a);
#pragma unroll
            for (int i = 0; i < 8; i++) {
              acc[0][r] = fmaf(a[i], w0[i], acc[0][r]);
              acc[1][r] = fmaf(a[i], w1[i], acc[1][r]);
              if (GATED) {
                acu[0][r] = fmaf(a[i], u0[i], acu[0][r]);
                acu[1][r] = fmaf(a[i], u1[i], acu[1][r]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < GV_ROWS; r++) {
        if (r < nr) {
#pragma unroll
          for (int j = 0; j < 2; j++) {
            float v = warp_sum(acc[j][r]);
            if (GATED) {
              const float u = warp_sum(acu[j][r]);
              v = ACT == ACT_CLAMPED ? clamped_unit(v, u, limit, alpha) : v / (1.f + expf(-v)) * u;
            }
            if (ACT == ACT_GELU) v = gelu_erf_f(v);
            const int f = f0 + j;
            if (lane == 0 && f < N) C[(size_t)(r0 + r) * ldc + f] = from_float<TC>(v);
          }
        }
      }
    }
  }
}

// out[t] = sum_k top_w[t, k] * y[place_of[t * top + k]]  (+ shared[t]), in choice order, float32 sums, rounded once.
// shared: [rows, H] in the activation type, or float32 slices [n_slices][rows, H] added in slice order; shared_gate
// (float32 [rows], or null): the shared part is multiplied by sigmoid(shared_gate[t]) before it is added.
template <typename T, typename TY>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ place_of,
                                   const float* __restrict__ top_w, const T* __restrict__ shared_t,
                                   const float* __restrict__ shared_slices, int n_slices, long long slice_stride,
                                   T* __restrict__ out, int H, int top, const float* __restrict__ shared_gate) {
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const float sg = shared_gate != nullptr ? 1.f / (1.f + expf(-shared_gate[t])) : 1.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; k++) {
      const int p = place_of[(size_t)t * top + k];
      if (p >= 0) acc = fmaf(top_w[(size_t)t * top + k], to_float(y[(size_t)p * H + i]), acc);
    }
    if (shared_gate == nullptr) {
      if (shared_t != nullptr) acc += to_float(shared_t[(size_t)t * H + i]);
      for (int s = 0; s < n_slices; s++) acc += shared_slices[(size_t)s * slice_stride + (size_t)t * H + i];
    } else {
      float sh = shared_t != nullptr ? to_float(shared_t[(size_t)t * H + i]) : 0.f;
      for (int s = 0; s < n_slices; s++) sh += shared_slices[(size_t)s * slice_stride + (size_t)t * H + i];
      acc = fmaf(sg, sh, acc);
    }
    out[(size_t)t * H + i] = from_float<T>(acc);
  }
}

template <typename T>
int route_launch(const void* h, const float* wr, const float* br, const int* token_seq, int* top_idx, float* top_w,
                 float* logits, int n_tokens, int H, int E, int top, int over_all, float scale, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || (size_t)E * 4 * ROUTE_WARPS > 48 * 1024 || (E + 3) / 4 > 65535) return -2;
  const int tb = (n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS;
  int rc = launch_pdl(moe_logits_kernel<T>, dim3(tb, (E + 3) / 4), dim3(ROUTE_WARPS * 32), 0, st, (const T*)h, wr, br,
                      logits, n_tokens, H, E);
  if (rc != 0) return rc;
  return launch_pdl(moe_choose_kernel, dim3(tb), dim3(ROUTE_WARPS * 32), (size_t)ROUTE_WARPS * E * sizeof(float), st,
                    (const float*)logits, token_seq, top_idx, top_w, n_tokens, E, top, over_all, scale);
}

template <typename T>
int route_scored_launch(const void* h, const float* wr, const float* br, const float* correction, const int* token_seq,
                        int* top_idx, float* top_w, float* logits, int n_tokens, int H, int E, int top, int groups,
                        int keep, float scale, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
      top > keep * (E / groups) || (size_t)(2 * E + groups) * 4 * ROUTE_WARPS > 48 * 1024 || (E + 3) / 4 > 65535)
    return -2;
  const int tb = (n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS;
  int rc = launch_pdl(moe_logits_kernel<T>, dim3(tb, (E + 3) / 4), dim3(ROUTE_WARPS * 32), 0, st, (const T*)h, wr, br,
                      logits, n_tokens, H, E);
  if (rc != 0) return rc;
  return launch_pdl(moe_choose_scored_kernel, dim3(tb), dim3(ROUTE_WARPS * 32),
                    (size_t)ROUTE_WARPS * (2 * E + groups) * sizeof(float), st, (const float*)logits, correction,
                    token_seq, top_idx, top_w, n_tokens, E, top, groups, keep, scale);
}

template <typename TA, typename TC, int ACT>
int gemm_launch(const void* A, int lda, const void* W, void* C, int ldc, const int* offsets, const int* order, int top,
                int n_places, int E, int N, int K, cudaStream_t st, float limit = 0.f, float alpha = 0.f) {
  if (n_places <= 0 || N <= 0) return 0;
  if (K <= 0 || E <= 0) return -2;
  // few rows: every weight once, at full width (rows of 8 values must start on 16 bytes)
  const bool wide = K % 8 == 0 && lda % 8 == 0 && (((uintptr_t)A) & 15) == 0 && (((uintptr_t)W) & 15) == 0;
  if (wide && n_places <= GEMV_PLACES_MAX && E <= 65535)
    return launch_pdl(moe_gemv_kernel<TA, TC, ACT>, dim3((N + GV_FEATS - 1) / GV_FEATS, E), dim3(GV_WARPS * 32), 0, st,
                      (const TA*)A, lda, (const TA*)W, (TC*)C, ldc, offsets, order, top, N, K, limit, alpha);
  const int row_tiles = n_places / BM + E;  // sum over experts of ceil(count / BM) is at most this
  if (row_tiles > 65535) return -3;
  return launch_pdl(moe_gemm_kernel<TA, TC, ACT>, dim3((N + BN - 1) / BN, row_tiles), dim3(256), 0, st, (const TA*)A,
                    lda, (const TA*)W, (TC*)C, ldc, offsets, order, top, E, N, K, limit, alpha);
}

template <typename T, typename TY>
int combine_launch(const void* y, const int* place_of, const float* top_w, const void* shared_t,
                   const float* shared_slices, int n_slices, long long slice_stride, void* out, int n_tokens, int H,
                   int top, const float* shared_gate, cudaStream_t st) {
  if (n_tokens <= 0) return 0;
  return launch_pdl(moe_combine_kernel<T, TY>, dim3(n_tokens), dim3(H >= 1024 ? 256 : 128), 0, st, (const TY*)y, place_of, top_w,
                    (const T*)shared_t, shared_slices, n_slices, slice_stride, (T*)out, H, top, shared_gate);
}

}  // namespace

TKB_EXPORT int tkb_moe_order(const int* top_idx, int n_pairs, int E, int top, int pad, int* offsets, int* order,
                             int* place_of, int* tile_group, int n_tiles, int* src_token, int cap, void* st) {
  if (n_pairs <= 0) return 0;
  if (E <= 0 || top <= 0 || pad <= 0 || (size_t)(3 * E + 1) * 4 > 48 * 1024) return -2;
  return launch_pdl(moe_order_kernel, dim3(1), dim3(1024), (size_t)(3 * E + 1) * sizeof(int), (cudaStream_t)st, top_idx,
                    n_pairs, E, top, pad, offsets, order, place_of, tile_group, n_tiles, src_token, cap);
}

#define TKB_MOE_EXPORTS(SUF, T)                                                                                        \
  TKB_EXPORT int tkb_moe_route_##SUF(const void* h, const float* wr, const float* br, const int* token_seq,            \
                                     int* top_idx, float* top_w, float* logits, int n_tokens, int H, int E, int top,   \
                                     int over_all, float scale, void* st) {                                            \
    return route_launch<T>(h, wr, br, token_seq, top_idx, top_w, logits, n_tokens, H, E, top, over_all, scale,         \
                           (cudaStream_t)st);                                                                          \
  }                                                                                                                    \
  TKB_EXPORT int tkb_moe_logits_##SUF(const void* h, const float* wr, const float* br, float* logits, int n_tokens,    \
                                      int H, int E, void* st) {                                                        \
    if (n_tokens <= 0) return 0;                                                                                       \
    if (E <= 0 || (E + 3) / 4 > 65535) return -2;                                                                      \
    return launch_pdl(moe_logits_kernel<T>, dim3((n_tokens + ROUTE_WARPS - 1) / ROUTE_WARPS, (E + 3) / 4),             \
                      dim3(ROUTE_WARPS * 32), 0, (cudaStream_t)st, (const T*)h, wr, br, logits, n_tokens, H, E);       \
  }                                                                                                                    \
  TKB_EXPORT int tkb_moe_gemm_gated_##SUF(const void* A, int lda, const void* W, void* C, int ldc, const int* offsets, \
                                          const int* order, int top, int n_places, int E, int N, int K, void* st) {    \
    return gemm_launch<T, T, ACT_GATED>(A, lda, W, C, ldc, offsets, order, top, n_places, E, N, K, (cudaStream_t)st);  \
  }                                                                                                                    \
  TKB_EXPORT int tkb_moe_gemm_clamped_##SUF(const void* A, int lda, const void* W, void* C, int ldc,                   \
                                            const int* offsets, const int* order, int top, int n_places, int E, int N, \
                                            int K, float limit, float alpha, void* st) {                               \
    if (!(limit > 0.f)) return -2;                                                                                     \
    return gemm_launch<T, T, ACT_CLAMPED>(A, lda, W, C, ldc, offsets, order, top, n_places, E, N, K, (cudaStream_t)st, \
                                          limit, alpha);                                                               \
  }                                                                                                                    \
  TKB_EXPORT int tkb_moe_gemm_gelu_##SUF(const void* A, int lda, const void* W, void* C, int ldc, const int* offsets,  \
                                         const int* order, int top, int n_places, int E, int N, int K, void* st) {     \
    return gemm_launch<T, T, ACT_GELU>(A, lda, W, C, ldc, offsets, order, top, n_places, E, N, K, (cudaStream_t)st);   \
  }                                                                                                                    \
  TKB_EXPORT int tkb_moe_route_scored_##SUF(const void* h, const float* wr, const float* br, const float* correction,  \
                                            const int* token_seq, int* top_idx, float* top_w, float* logits,           \
                                            int n_tokens, int H, int E, int top, int groups, int keep, float scale,    \
                                            void* st) {                                                                \
    return route_scored_launch<T>(h, wr, br, correction, token_seq, top_idx, top_w, logits, n_tokens, H, E, top,       \
                                  groups, keep, scale, (cudaStream_t)st);                                              \
  }                                                                                                                    \
  TKB_EXPORT int tkb_moe_gemm_##SUF(const void* A, int lda, const void* W, void* C, int ldc, const int* offsets,       \
                                    const int* order, int top, int n_places, int E, int N, int K, void* st) {          \
    return gemm_launch<T, float, ACT_NONE>(A, lda, W, C, ldc, offsets, order, top, n_places, E, N, K,                  \
                                           (cudaStream_t)st);                                                          \
  }                                                                                                                    \
  TKB_EXPORT int tkb_moe_combine_##SUF(const float* y, const int* place_of, const float* top_w, const void* shared_t,  \
                                       const float* shared_slices, int n_slices, long long slice_stride, void* out,    \
                                       int n_tokens, int H, int top, const float* shared_gate, void* st) {             \
    return combine_launch<T, float>(y, place_of, top_w, shared_t, shared_slices, n_slices, slice_stride, out, n_tokens, \
                                    H, top, shared_gate, (cudaStream_t)st);                                            \
  }                                                                                                                    \
  TKB_EXPORT int tkb_moe_gather_##SUF(const void* src, const int* src_token, void* dst, int n_places, int H,           \
                                      void* st) {                                                                      \
    if (n_places <= 0) return 0;                                                                                       \
    return launch_pdl(moe_gather_kernel<T>, dim3(n_places), dim3(H >= 1024 ? 256 : 128), 0, (cudaStream_t)st,          \
                      (const T*)src, src_token, (T*)dst, H);                                                           \
  }

TKB_MOE_EXPORTS(f32, float)
TKB_MOE_EXPORTS(bf16, __nv_bfloat16)

// The same weighted sum over expert outputs kept in bfloat16 (the tensor-core products' result).
TKB_EXPORT int tkb_moe_combine_y16_bf16(const void* y, const int* place_of, const float* top_w, const void* shared_t,
                                        const float* shared_slices, int n_slices, long long slice_stride, void* out,
                                        int n_tokens, int H, int top, const float* shared_gate, void* st) {
  return combine_launch<__nv_bfloat16, __nv_bfloat16>(y, place_of, top_w, shared_t, shared_slices, n_slices, slice_stride,
                                                      out, n_tokens, H, top, shared_gate, (cudaStream_t)st);
}

// ... and its sum as float32 rows, for a consumer that reads float32 (a norm).
TKB_EXPORT int tkb_moe_combine_y16_f32(const void* y, const int* place_of, const float* top_w, const void* shared_t,
                                       const float* shared_slices, int n_slices, long long slice_stride, void* out,
                                       int n_tokens, int H, int top, const float* shared_gate, void* st) {
  return combine_launch<float, __nv_bfloat16>(y, place_of, top_w, shared_t, shared_slices, n_slices, slice_stride, out,
                                              n_tokens, H, top, shared_gate, (cudaStream_t)st);
}
