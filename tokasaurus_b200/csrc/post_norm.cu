// Kernels of blocks that normalise a sublayer's OUTPUT and add it to the residual stream, and of the parts that
// such models bring along:
//
//   scaled_norm_add   x += mult * scale[c] * w[c] * (y + bias)[c] / sqrt(mean((y + bias)^2) + eps)   (x float32, in
//                     place), and the new x in the activation type for the sublayer that reads it next; y whole
//                     rows or the float32 slices of a K-split product
//   cast_rows         float32 rows in the activation type
//   add_sinusoid      x[t][2i] += sin(p_t * f_i),  x[t][2i+1] += cos(p_t * f_i)   (f_i a float64 table)
//   clamped_glu       g = min(gate, L), u = clamp(up, -L, L), out = g * sigmoid(alpha * g) * (u + 1)
//   gated_group_norm  a row of float32 values, gated and RMS-normed in equal parts:
//                       mode 0: out = N(y) * w * sigmoid(gate)        (the norm first)
//                       mode 1: out = N(y * silu(gate)) * w           (the gate first)
//                       mode 2: out = N(y) * w * silu(gate)           (the norm first, the gate a SiLU)
//                     w may be shorter than a row (one weight vector that every part shares) or absent
//   sum_group_norm    x = w * N_g(a * x + y): the norm AFTER the residual sum, in g equal parts of a row (x float32,
//                     in place; the new x also in the activation type); y float32 rows, float32 slices of a K-split
//                     product, or rows in the activation type
//   gelu_gate_rows    out[r][j] = gelu_tanh(z[r][j]) * table[token(r)][off + j]: a gate times a slice of a second
//                     embedding table, the token's id resolved like the embedding's
//
// Statistics, sums and the residual stream are float32 whatever the activation type.  One block a row.
#include "common.cuh"

using namespace tkb;

namespace {

inline int row_threads(int n) {
  int t = 32;
  while (t < n / 4 && t < 512) t <<= 1;
  return t;
}

template <typename T>
__global__ void __launch_bounds__(512)
scaled_norm_add_kernel(float* __restrict__ x, const float* __restrict__ y, int n_slices, long long slice_stride,
                       const float* __restrict__ bias, const float* __restrict__ w, const float* __restrict__ scale,
                       float mult, float eps, T* __restrict__ h_out, int H) {
  __shared__ float red[33];
  trigger_dependents();
  grid_dependency_wait();
  const size_t row = (size_t)blockIdx.x * H;
  // y may arrive as the float32 slices of a K-split product: they are added in slice order, both times alike
  auto value = [&](int c) {
    float v = y[row + c];
    for (int s = 1; s < n_slices; s++) v += y[(size_t)s * slice_stride + row + c];
    return v + (bias ? bias[c] : 0.f);
  };
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = value(c);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = value(c);
    float u = v * r * w[c];
    if (scale) u *= scale[c];
    const float nx = fmaf(mult, u, x[row + c]);
    x[row + c] = nx;
    if (h_out) h_out[row + c] = from_float<T>(nx);
  }
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, size_t n) {
  trigger_dependents();
  grid_dependency_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_float<T>(x[i]);
}

// Frequencies, angle, sine and cosine in float64 (a float32 product of a position in the thousands and a frequency is off
// by 1e-4 of a radian); what is added to the row is their float32 rounding.
__global__ void add_sinusoid_kernel(float* __restrict__ x, const int* __restrict__ positions,
                                    const double* __restrict__ freq, int H) {
  trigger_dependents();
  grid_dependency_wait();
  const double p = (double)positions[blockIdx.x];
  float* row = x + (size_t)blockIdx.x * H;
  for (int i = threadIdx.x; 2 * i < H; i += blockDim.x) {
    double s, c;
    sincos(p * freq[i], &s, &c);
    row[2 * i] += (float)s;
    if (2 * i + 1 < H) row[2 * i + 1] += (float)c;
  }
}

// interleave 0: a row is [gate | up]; 8: columns in groups of 16, 8 gate columns then the 8 up columns of the same features
template <typename TI, typename TO>
__global__ void clamped_glu_kernel(const TI* __restrict__ gate_up, TO* __restrict__ out, int inner, float limit,
                                   float alpha, int interleave) {
  trigger_dependents();
  grid_dependency_wait();
  const TI* row = gate_up + (size_t)blockIdx.x * 2 * inner;
  TO* orow = out + (size_t)blockIdx.x * inner;
  for (int i = threadIdx.x; i < inner; i += blockDim.x) {
    const int gi = interleave ? ((i >> 3) << 4) + (i & 7) : i;
    const int ui = interleave ? gi + 8 : inner + i;
    const float g = fminf(to_float(row[gi]), limit);
    const float u = fminf(fmaxf(to_float(row[ui]), -limit), limit);
    orow[i] = from_float<TO>(g / (1.f + expf(-alpha * g)) * (u + 1.f));
  }
}


// x = w * N_g(a * x + y) with N_g dividing each of the row's equal parts by its own root mean square.  Block (row,
// part).  y: float32 rows (one or more slices, added in slice order) or rows in the activation type.
template <typename T>
__global__ void __launch_bounds__(512)
sum_group_norm_kernel(float* __restrict__ x, const float* __restrict__ y32, int n_slices, long long slice_stride,
                      const T* __restrict__ y_act, float a, const float* __restrict__ w, float eps,
                      T* __restrict__ h_out, int H, int part) {
  __shared__ float red[33];
  trigger_dependents();
  grid_dependency_wait();
  const size_t row = (size_t)blockIdx.x * H + (size_t)blockIdx.y * part;
  const int c0 = blockIdx.y * part;
  auto value = [&](int c) {
    float v = 0.f;
    if (y32 != nullptr) {
      v = y32[row + c];
      for (int s = 1; s < n_slices; s++) v += y32[(size_t)s * slice_stride + row + c];
    } else if (y_act != nullptr) {
      v = to_float(y_act[row + c]);
    }
    return fmaf(a, x[row + c], v);
  };
  float ss = 0.f;
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    const float v = value(c);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)part + eps);
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    const float nx = value(c) * r * w[c0 + c];
    x[row + c] = nx;  // (each thread reads and writes its own elements only)
    if (h_out) h_out[row + c] = from_float<T>(nx);
  }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// rows: the tokens whose rows z holds (null: row r is token r)
template <typename TZ, typename TE, typename TO>
__global__ void gelu_gate_rows_kernel(const TZ* __restrict__ z, const TE* __restrict__ table, int table_stride, int off,
                                      int dim, int V, const int* __restrict__ ids, const int* __restrict__ token_seq,
                                      const int* __restrict__ seq_slot, const int* __restrict__ last_token,
                                      const int* __restrict__ rows, TO* __restrict__ out, int* __restrict__ status) {
  trigger_dependents();
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  const int s = token_seq[t];
  int id = ids[t];
  bool valid = s >= 0;
  if (valid && id < 0) id = last_token[seq_slot[s]];
  if (valid && (id < 0 || id >= V)) {
    if (threadIdx.x == 0) atomicOr(status, TKB_STATUS_BAD_TOKEN_ID);
    valid = false;
  }
  TO* orow = out + (size_t)r * dim;
  for (int j = threadIdx.x; j < dim; j += blockDim.x)
    orow[j] = from_float<TO>(valid ? gelu_tanh_f(to_float(z[(size_t)r * dim + j])) *
                                         to_float(table[(size_t)id * table_stride + off + j])
                                   : 0.f);
}

// One block a (row, part).  mode 1: the values are multiplied by silu(gate) before the statistics; modes 0 and 2: the
// normed values are multiplied by sigmoid(gate) or silu(gate).  w holds w_len weights, used round and round (w_len = the
// row's width: a weight for every value); null: none.
template <typename T>
__global__ void __launch_bounds__(512)
gated_group_norm_kernel(const float* __restrict__ y, int y_stride, const float* __restrict__ gate, int gate_stride,
                        const float* __restrict__ w, int w_len, T* __restrict__ out, int out_stride, int part, float eps,
                        int mode) {
  __shared__ float red[33];
  trigger_dependents();
  grid_dependency_wait();
  const int c0 = blockIdx.y * part;
  const float* yr = y + (size_t)blockIdx.x * y_stride + c0;
  const float* gr = gate + (size_t)blockIdx.x * gate_stride + c0;
  const bool gate_first = mode == 1;
  float ss = 0.f;
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    float v = yr[c];
    if (gate_first) {
      const float g = gr[c];
      v *= g / (1.f + expf(-g));
    }
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float r = rsqrtf(ss / (float)part + eps);
  T* orow = out + (size_t)blockIdx.x * out_stride + c0;
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    float v = yr[c];
    const float g = gr[c];
    const float wc = w ? w[(c0 + c) % w_len] : 1.f;
    if (gate_first) v = v * (g / (1.f + expf(-g))) * r * wc;
    else if (mode == 2) v = v * r * wc * (g / (1.f + expf(-g)));
    else v = v * r * wc / (1.f + expf(-g));
    orow[c] = from_float<T>(v);
  }
}

}  // namespace

#define TKB_POST_NORM_EXPORTS(SUF, T)                                                                                 \
  TKB_EXPORT int tkb_scaled_norm_add_##SUF(float* x, const float* y, int n_slices, long long slice_stride,            \
                                           const float* bias, const float* w, const float* scale, float mult,         \
                                           float eps, void* h_out, int rows, int H, void* st) {                       \
    if (rows <= 0) return 0;                                                                                          \
    if (H <= 0 || n_slices < 1) return -2;                                                                            \
    return launch_pdl(scaled_norm_add_kernel<T>, dim3(rows), dim3(row_threads(H)), 0, (cudaStream_t)st, x, y,         \
                      n_slices, slice_stride, bias, w, scale, mult, eps, (T*)h_out, H);                               \
  }                                                                                                                   \
  TKB_EXPORT int tkb_cast_rows_##SUF(const float* x, void* out, long long n, void* st) {                              \
    if (n <= 0) return 0;                                                                                             \
    const long long blocks = (n + 1023) / 1024;                                                                       \
    return launch_pdl(cast_rows_kernel<T>, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0,             \
                      (cudaStream_t)st, x, (T*)out, (size_t)n);                                                       \
  }                                                                                                                   \
  TKB_EXPORT int tkb_gated_group_norm_##SUF(const float* y, int y_stride, const float* gate, int gate_stride,         \
                                            const float* w, int w_len, void* out, int out_stride, int rows,           \
                                            int width, int groups, float eps, int mode, void* st) {                   \
    if (rows <= 0) return 0;                                                                                          \
    if (groups <= 0 || width <= 0 || width % groups || (w != nullptr && w_len <= 0) || mode < 0 || mode > 2)          \
      return -2;                                                                                                      \
    if (groups > 65535) return -3;                                                                                    \
    return launch_pdl(gated_group_norm_kernel<T>, dim3(rows, groups), dim3(row_threads(width / groups)), 0,           \
                      (cudaStream_t)st, y, y_stride, gate, gate_stride, w, w_len, (T*)out, out_stride,                \
                      width / groups, eps, mode);                                                                     \
  }                                                                                                                   \
  TKB_EXPORT int tkb_sum_group_norm_##SUF(float* x, const float* y32, int n_slices, long long slice_stride,           \
                                          const void* y_act, float a, const float* w, float eps, void* h_out,         \
                                          int rows, int H, int groups, void* st) {                                    \
    if (rows <= 0) return 0;                                                                                          \
    if (H <= 0 || groups <= 0 || H % groups || (y32 != nullptr && n_slices < 1)) return -2;                           \
    if (groups > 65535) return -3;                                                                                    \
    return launch_pdl(sum_group_norm_kernel<T>, dim3(rows, groups), dim3(row_threads(H / groups)), 0,                 \
                      (cudaStream_t)st, x, y32, n_slices, slice_stride, (const T*)y_act, a, w, eps, (T*)h_out, H,     \
                      H / groups);                                                                                    \
  }

TKB_POST_NORM_EXPORTS(f32, float)
TKB_POST_NORM_EXPORTS(bf16, __nv_bfloat16)

TKB_EXPORT int tkb_add_sinusoid(float* x, const int* positions, const double* freq, int rows, int H, void* st) {
  if (rows <= 0) return 0;
  return launch_pdl(add_sinusoid_kernel, dim3(rows), dim3(row_threads(H * 2)), 0, (cudaStream_t)st, x, positions,
                    freq, H);
}

// gate_up [rows, 2 * inner] (gate columns, then up columns) in the activation type or float32; out [rows, inner]
#define TKB_GLU_EXPORT(NAME, TI, TO)                                                                                  \
  TKB_EXPORT int NAME(const void* gate_up, void* out, int rows, int inner, float limit, float alpha, int interleave,  \
                      void* st) {                                                                                     \
    if (rows <= 0) return 0;                                                                                          \
    if (inner <= 0 || (interleave != 0 && (interleave != 8 || inner % 8))) return -2;                                 \
    return launch_pdl(clamped_glu_kernel<TI, TO>, dim3(rows), dim3(row_threads(inner * 4)), 0, (cudaStream_t)st,      \
                      (const TI*)gate_up, (TO*)out, inner, limit, alpha, interleave);                                 \
  }
TKB_GLU_EXPORT(tkb_clamped_glu_f32_f32, float, float)
TKB_GLU_EXPORT(tkb_clamped_glu_f32_bf16, float, __nv_bfloat16)
TKB_GLU_EXPORT(tkb_clamped_glu_bf16_bf16, __nv_bfloat16, __nv_bfloat16)

// z [rows, dim] float32 or in the activation type; table [V, table_stride] in the weights' type; out [rows, dim]
#define TKB_GATE_ROWS_EXPORT(NAME, TZ, TE, TO)                                                                        \
  TKB_EXPORT int NAME(const void* z, const void* table, int table_stride, int off, int dim, int V, const int* ids,    \
                      const int* token_seq, const int* seq_slot, const int* last_token, const int* rows, void* out,   \
                      int n_rows, int* status, void* st) {                                                            \
    if (n_rows <= 0) return 0;                                                                                        \
    if (dim <= 0 || off < 0 || off + dim > table_stride) return -2;                                                   \
    return launch_pdl(gelu_gate_rows_kernel<TZ, TE, TO>, dim3(n_rows), dim3(row_threads(dim * 4)), 0,                 \
                      (cudaStream_t)st, (const TZ*)z, (const TE*)table, table_stride, off, dim, V, ids, token_seq,    \
                      seq_slot, last_token, rows, (TO*)out, status);                                                  \
  }
TKB_GATE_ROWS_EXPORT(tkb_gelu_gate_rows_f32, float, float, float)
TKB_GATE_ROWS_EXPORT(tkb_gelu_gate_rows_bf16, float, __nv_bfloat16, __nv_bfloat16)
