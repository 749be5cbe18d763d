// A linear recurrence with a matrix state per head and ONE decay number per head and token:
//
//     S_t = a_t S_(t-1) + (c_t k_t) v_t^T,        o_t = S_t^T q_t + D v_t
//
// (S is dim x vdim; k_t, q_t have dim entries, v_t has vdim).  Two mixers are instances of it:
//   * decayed linear attention: a_t = lambda_head (a constant), c_t = 1, D = 0, q, k, v = silu of the projections
//     (silu_cols, in place), one q and k per head;
//   * the selective state space (state-space duality form): a_t = exp(-exp(A_head) dt_t), c_t = dt_t, k = B, q = C
//     shared by the heads of a group, v = x, D a number per head; x, B and C come out of a causal convolution over
//     time with bias and SiLU, dt_t = softplus(dt_raw + dt_bias).
//   * gated linear attention: a DIFFERENT decay for every key channel, S_t = diag(f_t) S_(t-1) + k_t v_t^T, with
//     f_t = sigmoid(A2 (A1 h_t) + b)^(1/tau) made beforehand for all tokens (gla_gates, which also scales q);
//   * retention: a_t = lambda_head, q and k rotated by position and k scaled beforehand (rotate_scale).
// Everything here is float32: projections arrive as float32 rows, the state lives in the request's slot as S^T,
// state[slot][head][vdim][dim], and the outputs leave as float32 rows for the norm that follows.
//
// Kernels: ssm_prep (convolution + SiLU for every channel of [x | B | C], dt and the decay; one block a token; inputs
// from before the step come from the request's carried inputs), conv_carry (brings the carried inputs forward after
// every token has read them), decay_walk (the recurrence; a build of it with a decay vector a token and head),
// gla_gates, rotate_scale.
//
// The walk: one block owns some columns of the state of one (request, head) and goes over the request's tokens of
// this step in order.  LANES threads share a column j of S (lane L holds dims 4 (L + LANES i) .. + 3): a step is 2 DPT
// multiply-adds and a shuffle sum a thread.  A thread holds as little of the state as the head allows (four values at
// heads of 128): a warp alone issues an instruction every four cycles (each waits for the one before), so the time
// goes down with the number of warps, and that is the state's size over what a thread holds.  Tokens come in chunks of
// 16 by cp.async, one chunk ahead; the lanes' shares of a chunk's outputs wait in shared memory and are added up after
// the chunk.  Activations of q, k and v are applied beforehand, once.
//
// Compile with -DTKB_DR_LANES=<threads that share a column: the power of two from 8 to 32 nearest above dim / 4> and
// -DTKB_DR_DPT=<dims a lane: 4 * ceil(dim / (4 * lanes))>.
#include "common.cuh"

#ifndef TKB_DR_DPT
#error "compile with -DTKB_DR_DPT=<dims per thread>"
#endif
#ifndef TKB_DR_LANES
#error "compile with -DTKB_DR_LANES=<threads that share a column: 8, 16 or 32>"
#endif

using namespace tkb;

namespace {

constexpr int DPT = TKB_DR_DPT;
static_assert(DPT % 4 == 0 && DPT >= 4, "dims a lane: a multiple of 4");
constexpr int LANES = TKB_DR_LANES;
static_assert(LANES == 8 || LANES == 16 || LANES == 32, "8, 16 or 32 threads a column");
constexpr int CHUNK = 16;

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }
// log(1 + e^z); beyond 20 the sum is z itself in float32
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// proj: float32 [T, stride]; channels xbc_off .. xbc_off + C are convolved, columns dt_off .. dt_off + H are step sizes
__global__ void __launch_bounds__(512)
ssm_prep_kernel(const float* __restrict__ proj, int stride, int xbc_off, int C, int taps,
                const float* __restrict__ conv_w, const float* __restrict__ conv_b, const float* __restrict__ state,
                long long slot_stride, long long carry_off, const int* __restrict__ token_seq,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start, float* __restrict__ xbc,
                int dt_off, int H, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                float* __restrict__ dt_dec) {
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int s = token_seq[t];
  if (s < 0) return;
  const int i = t - seq_q_start[s];
  const float* carry = state + (size_t)seq_slot[s] * slot_stride + carry_off;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = conv_b ? conv_b[c] : 0.f;
    for (int j = 0; j < taps; j++) {
      const int back = taps - 1 - j;  // how many tokens before this one
      float u;
      if (i - back >= 0) u = proj[(size_t)(t - back) * stride + xbc_off + c];
      else u = carry[(size_t)(i + j) * C + c];
      acc = fmaf(conv_w[(size_t)c * taps + j], u, acc);
    }
    xbc[(size_t)t * C + c] = silu_f(acc);
  }
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float dt = softplus_f(proj[(size_t)t * stride + dt_off + h] + dt_bias[h]);
    dt_dec[(size_t)t * 2 * H + h] = dt;
    dt_dec[(size_t)t * 2 * H + H + h] = expf(-expf(a_log[h]) * dt);
  }
}

// One block a request: the last taps - 1 inputs of [carried inputs ; this step's inputs] become the carried inputs.
__global__ void __launch_bounds__(512)
conv_carry_kernel(const float* __restrict__ proj, int stride, int xbc_off, int C, int taps, float* __restrict__ state,
                  long long slot_stride, long long carry_off, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len) {
  trigger_dependents();
  grid_dependency_wait();
  const int s = blockIdx.x;
  const int n = seq_q_len[s];
  if (n <= 0) return;
  const int start = seq_q_start[s];
  float* carry = state + (size_t)seq_slot[s] * slot_stride + carry_off;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    for (int r = 0; r < taps - 1; r++) {  // ascending: row n + r is read before it is written
      const int at = n + r;               // index in [carried ; new]
      carry[(size_t)r * C + c] = at < taps - 1 ? carry[(size_t)at * C + c]
                                               : proj[(size_t)(start + at - (taps - 1)) * stride + xbc_off + c];
    }
  }
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// SiLU in place on `ncols` columns of float32 rows (the projections of a mixer whose q, k and v pass through it): done
// once for all tokens, not by every block that walks over them.
__global__ void silu_cols_kernel(float* __restrict__ x, int stride, int ncols) {
  trigger_dependents();
  grid_dependency_wait();
  float* row = x + (size_t)blockIdx.x * stride;
  for (int c = threadIdx.x; c < ncols; c += blockDim.x) row[c] = silu_f(row[c]);
}

// Shared memory of the walk, per buffer: q and k rows of QROW floats as they lie in memory (lane L reads the 16-byte
// pieces L, L + LANES, ...: the lanes of a column read neighbouring pieces, so no bank is hit twice), v at `cols` floats
// a token, decay and key scale a float a token each.
constexpr int QROW = LANES * DPT;

// VEC: a decay for every key channel, fvec [T, heads * dim] rows of f_stride floats, staged beside q and k.
template <bool VEC>
__global__ void __launch_bounds__(1024)
decay_walk_kernel(const float* __restrict__ q, int q_stride, const float* __restrict__ k, int k_stride, int qk_div,
                  const float* __restrict__ fvec, int f_stride,
                  const float* __restrict__ v, int v_stride, const float* __restrict__ dt_dec,
                  const float* __restrict__ decay_head, const float* __restrict__ skip, float* __restrict__ state,
                  long long slot_stride, float* __restrict__ out, const int* __restrict__ seq_slot,
                  const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len, int heads, int dim, int vdim,
                  int write_state, int cols_per_block, int vec_qk, int vec_v, int vec_s, int chunk) {
  extern __shared__ __align__(16) float smem[];
  const int cols = min(cols_per_block, vdim);
  const int cols4 = (cols + 3) & ~3;
  constexpr int NQ = VEC ? 3 : 2;  // staged rows of QROW floats a token: q, k (and the decays)
  const int buf_floats = chunk * (NQ * QROW + cols4 + 2);
  float* os = smem + 2 * buf_floats;  // the lanes' shares of a chunk's outputs: [cols][LANES][chunk + 1]
  const int orow = chunk + 1;         // (one float of padding: the lanes of a column write different banks)
  const int s = blockIdx.x, head = blockIdx.y;
  const int n = seq_q_len[s];
  if (n <= 0) return;
  const int start = seq_q_start[s];
  const int tid = threadIdx.x, lane = tid & (LANES - 1);
  const int col_begin = blockIdx.z * cols_per_block;
  const int col_end = min(vdim, col_begin + cols_per_block);
  if (col_begin >= col_end) return;
  const int ncols = col_end - col_begin;
  const int lc = tid / LANES;  // this thread's column within the block
  const int j = col_begin + lc;
  // dims beyond `dim` of the last lanes are read: zero the buffers once if there are any (the copies never touch them)
  if (dim < LANES * DPT)
    for (int idx = tid; idx < 2 * buf_floats; idx += blockDim.x) smem[idx] = 0.f;
  grid_dependency_wait();
  float* st = state + (size_t)seq_slot[s] * slot_stride + (size_t)head * vdim * dim;

  float S[DPT];
  if (vec_s) {
#pragma unroll
    for (int i = 0; i < DPT; i += 4) {
      const int d = 4 * (lane + LANES * (i >> 2));
      const float4 x = (j < col_end && d < dim) ? *reinterpret_cast<const float4*>(st + (size_t)j * dim + d)
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
      S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < DPT; i++) {
      const int d = 4 * (lane + LANES * (i >> 2)) + (i & 3);
      S[i] = (j < col_end && d < dim) ? st[(size_t)j * dim + d] : 0.f;
    }
  }
  const float* qh = q + (size_t)(head / qk_div) * dim;
  const float* kh = k + (size_t)(head / qk_div) * dim;
  const float* fh = VEC ? fvec + (size_t)head * dim : nullptr;
  const float* vh = v + (size_t)head * vdim + col_begin;
  const float a_const = decay_head ? decay_head[head] : 1.f;
  const float d_skip = skip ? skip[head] : 0.f;
  __syncthreads();  // the zeros are in place before the first copies land

  auto stage = [&](int t0, int b) {
    float* qs = smem + b * buf_floats;
    float* ks = qs + chunk * QROW;
    float* fs = ks + chunk * QROW;  // (VEC only)
    float* vs = qs + NQ * chunk * QROW;
    float* as = vs + chunk * cols4;
    float* cs = as + chunk;
    const int nt = min(chunk, n - t0);
    if (vec_qk) {
      const int d4n = dim >> 2;
      for (int idx = tid; idx < nt * d4n; idx += blockDim.x) {
        const int t = idx / d4n, d4 = idx - t * d4n;
        cp_async16(qs + t * QROW + 4 * d4, qh + (size_t)(start + t0 + t) * q_stride + 4 * d4);
        cp_async16(ks + t * QROW + 4 * d4, kh + (size_t)(start + t0 + t) * k_stride + 4 * d4);
        if (VEC) cp_async16(fs + t * QROW + 4 * d4, fh + (size_t)(start + t0 + t) * f_stride + 4 * d4);
      }
    } else {
      for (int idx = tid; idx < nt * dim; idx += blockDim.x) {
        const int t = idx / dim, d = idx - t * dim;
        cp_async4(qs + t * QROW + d, qh + (size_t)(start + t0 + t) * q_stride + d);
        cp_async4(ks + t * QROW + d, kh + (size_t)(start + t0 + t) * k_stride + d);
        if (VEC) cp_async4(fs + t * QROW + d, fh + (size_t)(start + t0 + t) * f_stride + d);
      }
    }
    if (vec_v && (ncols & 3) == 0) {
      const int c4n = ncols >> 2;
      for (int idx = tid; idx < nt * c4n; idx += blockDim.x) {
        const int t = idx / c4n, jj = (idx - t * c4n) * 4;
        cp_async16(vs + t * cols4 + jj, vh + (size_t)(start + t0 + t) * v_stride + jj);
      }
    } else {
      for (int idx = tid; idx < nt * ncols; idx += blockDim.x) {
        const int t = idx / ncols, jj = idx - t * ncols;
        cp_async4(vs + t * cols4 + jj, vh + (size_t)(start + t0 + t) * v_stride + jj);
      }
    }
    if (dt_dec != nullptr) {
      for (int t = tid; t < nt; t += blockDim.x) {
        cp_async4(cs + t, dt_dec + (size_t)(start + t0 + t) * 2 * heads + head);
        cp_async4(as + t, dt_dec + (size_t)(start + t0 + t) * 2 * heads + heads + head);
      }
    }
    cp_async_commit();
  };

  stage(0, 0);
  int b = 0;
  for (int t0 = 0; t0 < n; t0 += chunk, b ^= 1) {
    const int nt = min(chunk, n - t0);
    if (t0 + chunk < n) {
      stage(t0 + chunk, b ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* qs = smem + b * buf_floats;
    const float* ks = qs + chunk * QROW;
    const float* fs = ks + chunk * QROW;
    const float* vs = qs + NQ * chunk * QROW;
    const float* as = vs + chunk * cols4;
    const float* cs = as + chunk;
    float* mine = os + (lc * LANES + lane) * orow;
#pragma unroll 4
    for (int t = 0; t < nt; t++) {
      const float a = dt_dec ? as[t] : a_const, ck = dt_dec ? cs[t] : 1.f;
      const float4* q4 = reinterpret_cast<const float4*>(qs + t * QROW) + lane;
      const float4* k4 = reinterpret_cast<const float4*>(ks + t * QROW) + lane;
      const float4* f4 = reinterpret_cast<const float4*>(fs + t * QROW) + lane;
      const float vj = lc < ncols ? vs[t * cols4 + lc] : 0.f;
      const float cv = ck * vj;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int i = 0; i < DPT / 4; i++) {
        const float4 qq = q4[LANES * i], kk = k4[LANES * i];
        if (VEC) {
          const float4 ff = f4[LANES * i];
          S[4 * i + 0] = fmaf(ff.x, S[4 * i + 0], kk.x * cv);
          S[4 * i + 1] = fmaf(ff.y, S[4 * i + 1], kk.y * cv);
          S[4 * i + 2] = fmaf(ff.z, S[4 * i + 2], kk.z * cv);
          S[4 * i + 3] = fmaf(ff.w, S[4 * i + 3], kk.w * cv);
        } else {
          S[4 * i + 0] = fmaf(a, S[4 * i + 0], kk.x * cv);
          S[4 * i + 1] = fmaf(a, S[4 * i + 1], kk.y * cv);
          S[4 * i + 2] = fmaf(a, S[4 * i + 2], kk.z * cv);
          S[4 * i + 3] = fmaf(a, S[4 * i + 3], kk.w * cv);
        }
        a0 = fmaf(S[4 * i + 0], qq.x, a0);
        a1 = fmaf(S[4 * i + 1], qq.y, a1);
        a2 = fmaf(S[4 * i + 2], qq.z, a2);
        a3 = fmaf(S[4 * i + 3], qq.w, a3);
      }
      // this lane's share of o_t goes to shared memory; the shares are added up after the chunk (a shuffle sum here
      // would make every token wait for five dependent shuffles)
      const float acc = (a0 + a1) + (a2 + a3);
      mine[t] = lane == 0 ? fmaf(d_skip, vj, acc) : acc;
    }
    __syncwarp();  // a column's lanes are one warp, or part of one: its shares are all there
    // add the shares up: the lanes of a column split the chunk's tokens among them
    if (lc < ncols) {
      float* col_out = out + (size_t)(start + t0) * heads * vdim + (size_t)head * vdim + j;
      const float* shares = os + (size_t)lc * LANES * orow;
      if (LANES == 32 && chunk == 16) {
        const int t = lane & 15, l0 = (lane >> 4) * 16;
        float sum = 0.f;
#pragma unroll
        for (int l = 0; l < 16; l++) sum += shares[(l0 + l) * orow + t];
        sum += __shfl_xor_sync(0xffffffffu, sum, 16);
        if (lane < 16 && t < nt) col_out[(size_t)t * heads * vdim] = sum;
      } else {
        for (int t = lane; t < nt; t += LANES) {
          float sum = 0.f;
#pragma unroll
          for (int l = 0; l < LANES; l++) sum += shares[l * orow + t];
          col_out[(size_t)t * heads * vdim] = sum;
        }
      }
    }
    __syncthreads();  // the chunk's buffer may be filled again (by the stage after next), the shares overwritten
  }
  trigger_dependents();  // only now: the blocks of the kernel behind would sit on the SMs for the whole walk
  if (write_state) {
    if (vec_s) {
#pragma unroll
      for (int i = 0; i < DPT; i += 4) {
        const int d = 4 * (lane + LANES * (i >> 2));
        if (j < col_end && d < dim)
          *reinterpret_cast<float4*>(st + (size_t)j * dim + d) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < DPT; i++) {
        const int d = 4 * (lane + LANES * (i >> 2)) + (i & 3);
        if (j < col_end && d < dim) st[(size_t)j * dim + d] = S[i];
      }
    }
  }
}

int walk_launch(const float* q, int q_stride, const float* k, int k_stride, int qk_div, const float* fvec, int f_stride,
                const float* v, int v_stride,
                const float* dt_dec, const float* decay_head, const float* skip, float* state, long long slot_stride,
                float* out, const int* seq_slot, const int* seq_q_start, const int* seq_q_len, int n_seqs, int n_tokens,
                int heads, int dim, int vdim, int write_state, cudaStream_t st) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (dim <= 0 || dim > DPT * LANES || vdim <= 0 || heads <= 0 || qk_div <= 0) return -2;
  if (heads > 65535) return -3;
  // blocks of 256 threads: every block stages the head's q and k for itself (thinner blocks would pay more for that),
  // and several fit an SM with their loads of the state in flight together.  A step in which no request brings more
  // than one token stages one token at a time.
  const int chunk = n_tokens > n_seqs ? CHUNK : 1;
  int cols_per_block = 256 / LANES;
  if (cols_per_block > vdim) cols_per_block = vdim;
  const int splits = (vdim + cols_per_block - 1) / cols_per_block;
  if (splits > 65535) return -3;
  const int threads = ((cols_per_block * LANES + 31) / 32) * 32;
  const int cols4 = (cols_per_block + 3) & ~3;
  const int nq = fvec != nullptr ? 3 : 2;
  const size_t smem = (size_t)(2 * chunk * (nq * QROW + cols4 + 2) + cols_per_block * LANES * (chunk + 1)) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = fvec != nullptr
                        ? cudaFuncSetAttribute(decay_walk_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                        : cudaFuncSetAttribute(decay_walk_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int vec_qk = dim % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && al16(q) && al16(k) &&
                     (fvec == nullptr || (f_stride % 4 == 0 && al16(fvec)));
  const int vec_v = vdim % 4 == 0 && v_stride % 4 == 0 && cols_per_block % 4 == 0 && al16(v);
  const int vec_s = dim % 4 == 0 && slot_stride % 4 == 0 && al16(state);
  // An ordinary launch, not a programmatic one: blocks that come onto the SMs while the kernel ahead still holds some of
  // them are placed where room happens to be, several to an SM, and this kernel's few long-lived blocks then run on a
  // part of the GPU (measured: 0.84 ms instead of 0.36 ms for 2,048 tokens of 16 heads).
  if (fvec != nullptr)
    decay_walk_kernel<true><<<dim3(n_seqs, heads, splits), dim3(threads), smem, st>>>(
        q, q_stride, k, k_stride, qk_div, fvec, f_stride, v, v_stride, dt_dec, decay_head, skip, state, slot_stride, out,
        seq_slot, seq_q_start, seq_q_len, heads, dim, vdim, write_state, cols_per_block, vec_qk, vec_v, vec_s, chunk);
  else
    decay_walk_kernel<false><<<dim3(n_seqs, heads, splits), dim3(threads), smem, st>>>(
        q, q_stride, k, k_stride, qk_div, fvec, f_stride, v, v_stride, dt_dec, decay_head, skip, state, slot_stride, out,
        seq_slot, seq_q_start, seq_q_len, heads, dim, vdim, write_state, cols_per_block, vec_qk, vec_v, vec_s, chunk);
  return launch_status();
}

}  // namespace

TKB_EXPORT int tkb_ssm_prep(const float* proj, int stride, int xbc_off, int C, int taps, const float* conv_w,
                            const float* conv_b, float* state, long long slot_stride, long long carry_off,
                            const int* token_seq, const int* seq_slot, const int* seq_q_start, const int* seq_q_len,
                            int n_tokens, int n_seqs, float* xbc, int dt_off, int H, const float* dt_bias,
                            const float* a_log, float* dt_dec, int write_state, void* st) {
  if (n_tokens <= 0) return 0;
  if (taps < 1 || C <= 0 || H <= 0) return -2;
  int threads = 32;
  while (threads < C && threads < 512) threads <<= 1;
  int rc = launch_pdl(ssm_prep_kernel, dim3(n_tokens), dim3(threads), 0, (cudaStream_t)st, proj, stride, xbc_off, C,
                      taps, conv_w, conv_b, (const float*)state, slot_stride, carry_off, token_seq, seq_slot,
                      seq_q_start, xbc, dt_off, H, dt_bias, a_log, dt_dec);
  if (rc != 0 || !write_state || taps < 2 || n_seqs <= 0) return rc;
  return launch_pdl(conv_carry_kernel, dim3(n_seqs), dim3(threads), 0, (cudaStream_t)st, proj, stride, xbc_off, C,
                    taps, state, slot_stride, carry_off, seq_slot, seq_q_start, seq_q_len);
}

// dt_dec: float32 [T, 2 * heads] (key scale, then decay) or null, then decay_head [heads] is the decay and the key
// scale is 1; or fvec [T, heads * dim] (rows of f_stride floats): a decay for every key channel, key scale 1 (then
// dt_dec and decay_head are null).  skip: [heads] or null.
TKB_EXPORT int tkb_decay_walk(const float* q, int q_stride, const float* k, int k_stride, int qk_div, const float* fvec,
                              int f_stride, const float* v, int v_stride, const float* dt_dec, const float* decay_head, const float* skip,
                              float* state, long long slot_stride, float* out, const int* seq_slot,
                              const int* seq_q_start, const int* seq_q_len, int n_seqs, int n_tokens, int heads, int dim,
                              int vdim, int write_state, void* st) {
  if (fvec != nullptr && (dt_dec != nullptr || qk_div != 1)) return -2;
  return walk_launch(q, q_stride, k, k_stride, qk_div, fvec, f_stride, v, v_stride, dt_dec, decay_head, skip, state, slot_stride, out,
                     seq_slot, seq_q_start, seq_q_len, n_seqs, n_tokens, heads, dim, vdim, write_state, (cudaStream_t)st);
}

TKB_EXPORT int tkb_silu_cols(float* x, int stride, int ncols, int rows, void* st) {
  if (rows <= 0 || ncols <= 0) return 0;
  int threads = 32;
  while (threads < ncols / 4 && threads < 512) threads <<= 1;
  return launch_pdl(silu_cols_kernel, dim3(rows), dim3(threads), 0, (cudaStream_t)st, x, stride, ncols);
}

namespace {

// Decays of gated linear attention for GT tokens a block: z[c] = b[c] + sum_r A2t[r][c] low[t][r] (A2t float32
// [rank, C], the transposed second factor; low = A1 h, rank columns of the projections), f = sigmoid(z)^(1/tau) =
// exp(log_sigmoid(z) / tau) with log_sigmoid(z) = min(z, 0) - log1p(exp(-|z|)); and q (q_cols columns at q_off of
// the same rows) times q_scale, in place.
// A block owns GT tokens and blockDim.x columns (grid: token groups x column tiles), a thread one column of all GT
// tokens: the second factor's values come sixteen rows at a time (sixteen loads in flight a thread; a thread that
// walked all of a row's columns one load after the other took the same 0.2 ms for 8 tokens as for 2,048), the tokens'
// low-rank rows lie in shared memory rank-major, so that GT / 4 16-byte reads bring one rank's values of all GT tokens
// to the whole warp (one 4-byte read a token and rank made shared memory the bound at thousands of tokens).  The sum
// over the rank runs in order, whatever the tiling.  GT = 8 at every step size: with 32 tokens a block (a quarter of
// the second factor's traffic out of the L2) 2,048 tokens took 73 us against 49 us.
template <int GT>
__global__ void __launch_bounds__(256)
gla_gates_kernel(float* __restrict__ proj, int stride, int low_off, int rank, const float* __restrict__ a2t,
                 const float* __restrict__ bias, float inv_tau, int C, float* __restrict__ f, int q_off, int q_cols,
                 float q_scale, int n_tokens) {
  static_assert(GT % 4 == 0, "whole float4 a rank");
  extern __shared__ __align__(16) float low[];  // [rank][GT], tokens past the step's last zero
  trigger_dependents();
  grid_dependency_wait();
  const int t0 = blockIdx.x * GT;
  const int nt = min(GT, n_tokens - t0);
  for (int idx = threadIdx.x; idx < GT * rank; idx += blockDim.x) {
    const int t = idx / rank, r = idx - t * rank;
    low[r * GT + t] = t < nt ? proj[(size_t)(t0 + t) * stride + low_off + r] : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c < C) {
    float z[GT];
    const float b = bias ? bias[c] : 0.f;
#pragma unroll
    for (int t = 0; t < GT; t++) z[t] = b;
    auto add = [&](float w, int r) {
#pragma unroll
      for (int j = 0; j < GT / 4; j++) {
        const float4 l4 = *reinterpret_cast<const float4*>(low + r * GT + 4 * j);
        z[4 * j] = fmaf(w, l4.x, z[4 * j]);
        z[4 * j + 1] = fmaf(w, l4.y, z[4 * j + 1]);
        z[4 * j + 2] = fmaf(w, l4.z, z[4 * j + 2]);
        z[4 * j + 3] = fmaf(w, l4.w, z[4 * j + 3]);
      }
    };
    int r = 0;
    for (; r + 16 <= rank; r += 16) {
      float w[16];
#pragma unroll
      for (int i = 0; i < 16; i++) w[i] = a2t[(size_t)(r + i) * C + c];
#pragma unroll
      for (int i = 0; i < 16; i++) add(w[i], r + i);
    }
    for (; r < rank; r++) add(a2t[(size_t)r * C + c], r);
#pragma unroll
    for (int t = 0; t < GT; t++)
      if (t < nt) f[(size_t)(t0 + t) * C + c] = expf((fminf(z[t], 0.f) - log1pf(expf(-fabsf(z[t])))) * inv_tau);
  }
  if (q_scale != 1.f) {
    // eight loads in flight a thread, then the eight stores (one value at a time, every round trip to memory waited for
    // the one before: 8 tokens took as long as the decays themselves)
    const int total = nt * q_cols, step = gridDim.y * blockDim.x;
    int idx = blockIdx.y * blockDim.x + threadIdx.x;
    for (; idx + 7 * step < total; idx += 8 * step) {
      float* at[8];
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int j = idx + i * step, t = j / q_cols;
        at[i] = proj + (size_t)(t0 + t) * stride + q_off + (j - t * q_cols);
        v[i] = *at[i];
      }
#pragma unroll
      for (int i = 0; i < 8; i++) *at[i] = v[i] * q_scale;
    }
    for (; idx < total; idx += step) {
      const int t = idx / q_cols;
      proj[(size_t)(t0 + t) * stride + q_off + (idx - t * q_cols)] *= q_scale;
    }
  }
}

// Rotation by position of the q and k heads of float32 rows, in place: the first rot_dims channels of a head, channel i
// paired with i + rot_dims / 2 (pairs == 0) or channel 2i with 2i + 1 (pairs != 0); (u, v) -> (u cos a - v sin a,
// v cos a + u sin a), a = position * freq[i].  The angle, sine and cosine are float64 (the float32 product of a
// position in the thousands and a frequency is off by 1e-4 of a radian), made once a token for all heads.  Then q
// times q_scale and k times k_scale.  One block a token.
__global__ void __launch_bounds__(256)
rotate_scale_kernel(float* __restrict__ proj, int stride, int q_off, int k_off, int heads, int dim, int rot_dims,
                    int pairs, const double* __restrict__ freq, const int* __restrict__ positions,
                    const int* __restrict__ token_seq, float q_scale, float k_scale) {
  extern __shared__ float cs[];  // [rot_dims / 2] cosines, then as many sines
  trigger_dependents();
  grid_dependency_wait();
  const int t = blockIdx.x;
  if (token_seq[t] < 0) return;
  const int half = rot_dims / 2;
  const double p = (double)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double s, c;
    sincos(p * freq[i], &s, &c);
    cs[i] = (float)c;
    cs[half + i] = (float)s;
  }
  __syncthreads();
  float* row = proj + (size_t)t * stride;
  const int per_head = dim - half;  // a thread's items a head: `half` pairs, then the channels that pass
  for (int idx = threadIdx.x; idx < 2 * heads * per_head; idx += blockDim.x) {
    const int which = idx / (heads * per_head);
    const int rem = idx - which * heads * per_head;
    const int h = rem / per_head, i = rem - h * per_head;
    float* x = row + (which ? k_off : q_off) + (size_t)h * dim;
    const float sc = which ? k_scale : q_scale;
    if (i < half) {
      const int a = pairs ? 2 * i : i, b = pairs ? 2 * i + 1 : i + half;
      const float u = x[a], v = x[b], c = cs[i], s = cs[half + i];
      x[a] = (u * c - v * s) * sc;
      x[b] = (v * c + u * s) * sc;
    } else if (sc != 1.f) {
      x[rot_dims + (i - half)] *= sc;
    }
  }
}

}  // namespace

TKB_EXPORT int tkb_gla_gates(float* proj, int stride, int low_off, int rank, const float* a2t, const float* bias,
                             float inv_tau, int C, float* f, int q_off, int q_cols, float q_scale, int n_tokens,
                             void* st) {
  if (n_tokens <= 0) return 0;
  if (rank <= 0 || C <= 0 || (size_t)8 * rank * sizeof(float) > 48 * 1024) return -2;
  if ((C + 255) / 256 > 65535) return -2;
  return launch_pdl(gla_gates_kernel<8>, dim3((n_tokens + 7) / 8, (C + 255) / 256), dim3(256),
                    (size_t)8 * rank * sizeof(float), (cudaStream_t)st, proj, stride, low_off, rank, a2t, bias, inv_tau, C,
                    f, q_off, q_cols, q_scale, n_tokens);
}

TKB_EXPORT int tkb_rotate_scale(float* proj, int stride, int q_off, int k_off, int heads, int dim, int rot_dims,
                                int pairs, const double* freq, const int* positions, const int* token_seq,
                                float q_scale, float k_scale, int n_tokens, void* st) {
  if (n_tokens <= 0) return 0;
  if (heads <= 0 || dim <= 0 || rot_dims < 0 || rot_dims > dim || (rot_dims & 1) || (size_t)rot_dims * 4 > 48 * 1024)
    return -2;
  return launch_pdl(rotate_scale_kernel, dim3(n_tokens), dim3(256), (size_t)rot_dims * sizeof(float), (cudaStream_t)st,
                    proj, stride, q_off, k_off, heads, dim, rot_dims, pairs, freq, positions, token_seq, q_scale,
                    k_scale);
}
