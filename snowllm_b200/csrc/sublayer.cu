// Pieces of a layer whose norms sit on the sublayers' outputs, and of mixers that gate their heads.
//
//   norm_add:        residual += y / sqrt(mean(y^2) + eps) * w   (y: a sublayer's float output), and the
//                    sum again in the compute dtype: what the next sublayer reads
//   cast_rows:       the float residual in the compute dtype (the first sublayer's input)
//   gated_act:       out = act(gate) * up over [M, 2I] -> [M, I], act one of silu, relu, gelu (tanh form)
//   act_rows:        out = act(x), act one of silu, relu, gelu (tanh form), relu squared
//   rms_cols:        columns [off, off + n) of each row divided by their root mean square, times a weight
//   add_dyt:         residual += (a + b) for up to two float deltas (the second may be routed experts' outputs
//                    still in pieces), then the Dynamic Tanh norm tanh(alpha * x) * w + b of the sum: a norm
//                    without mean or variance
//   head_norm_gate:  per (row, head): o = a (- lambda * b), o / sqrt(mean(o^2) + eps) (* w) * mult
//                    * sigmoid(g) (or * silu(g)): the end of a mixer whose heads are normalised one by one and gated
//
// All statistics, sums and gates are evaluated in float; values are rounded to the compute dtype once,
// at the store.
#include "common.cuh"

enum { ACT_SILU = 0, ACT_RELU = 1, ACT_GELU_TANH = 2, ACT_RELU2 = 3 };

__device__ __forceinline__ float act_apply(float z, int act) {
  if (act == ACT_RELU) return fmaxf(z, 0.f);
  if (act == ACT_RELU2) {
    const float p = fmaxf(z, 0.f);
    return p * p;
  }
  if (act == ACT_GELU_TANH)
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return z / (1.f + expf(-z));
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// ---------------------------------------------------------------------------------------------
// One block per row.  The row of y is kept in shared memory between the two passes.
template <typename T>
__global__ void norm_add_kernel(float* __restrict__ residual, const float* __restrict__ y, SmallVec gamma,
                                T* __restrict__ x_out, int H, float eps) {
  pdl_begin();
  extern __shared__ __align__(16) float ys[];      // H floats + 33 for the reduction
  float* red = ys + ((H + 3) & ~3);
  const size_t r = blockIdx.x;
  const float* yr = y + r * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = yr[i];
    ys[i] = v;
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  float* res = residual + r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float v = res[i] + ys[i] * inv * gamma[i];
    res[i] = v;
    if (x_out) x_out[r * H + i] = from_f<T>(v);
  }
}

SNK_API int snk_norm_add(float* residual, const float* y, const void* gamma, int gamma_f32, void* x_out,
                         int M, int H, float eps, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (H <= 0) return SNK_ERR_SIZE;
  const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
  if (smem > 200 * 1024) return SNK_ERR_SIZE;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  SNK_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_add_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    snk_launch(norm_add_kernel<T>, dim3(M), dim3(threads), smem, stream, residual, y,
               SmallVec{gamma, gamma_f32}, static_cast<T*>(x_out), H, eps);
  });
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long long n) {
  pdl_begin();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = from_f<T>(x[i]);
}

SNK_API int snk_cast_rows(const float* x, void* out, long long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  SNK_DISPATCH(dtype, snk_launch(cast_rows_kernel<T>, dim3(blocks), dim3(256), 0, stream, x, static_cast<T*>(out), n));
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Columns of gate_up: (gate | up), or with `interleaved` blocks of 8 gate columns followed by the 8 up
// columns of the same features.
// act ACT_SWISH_CLAMP (the gated kind only): g = min(g, limit), u = clamp(u, -limit, limit), and the product is
// g * sigmoid(1.702 g) * (u + 1).
#define ACT_SWISH_CLAMP 4
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int M, int inter,
                                 int interleaved, int act, float limit) {
  pdl_begin();
  const long long n = (long long)M * inter;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long m = i / inter;
    const int c = (int)(i - m * inter);
    const T* row = gate_up + m * 2 * inter;
    float g, u;
    if (interleaved) {
      const int at = (c >> 3) * 16 + (c & 7);
      g = to_f<T>(row[at]);
      u = to_f<T>(row[at + 8]);
    } else {
      g = to_f<T>(row[c]);
      u = to_f<T>(row[inter + c]);
    }
    if (act == ACT_SWISH_CLAMP) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
      out[i] = from_f<T>(g / (1.f + expf(-1.702f * g)) * (u + 1.f));
    } else {
      out[i] = from_f<T>(act_apply(g, act) * u);
    }
  }
}

SNK_API int snk_gated_act(const void* gate_up, void* out, int M, int inter, int interleaved, int act, float limit,
                          int dtype, cudaStream_t stream) {
  if (M <= 0 || inter <= 0) return 0;
  if (act < 0 || act > ACT_SWISH_CLAMP || (interleaved && inter % 8)) return SNK_ERR_SIZE;
  if (act == ACT_SWISH_CLAMP && !(limit > 0.f)) return SNK_ERR_SIZE;
  const long long n = (long long)M * inter;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  SNK_DISPATCH(dtype, snk_launch(gated_act_kernel<T>, dim3(blocks), dim3(256), 0, stream,
                                 static_cast<const T*>(gate_up), static_cast<T*>(out), M, inter, interleaved, act,
                                 limit));
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// One warp per (row, head).  a: float [M, heads, a_stride] with the head's values in its first `dv`
// elements; with `second` the values to take off lie `second` elements further on (two maps of one
// head side by side).  g: the gate's pre-activation (float or bfloat16), row pitch g_ld, column
// h*dv + c.  w (may be null): a weight over heads*dv.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ a, int a_stride, int second, float lambda,
                                      SmallVec w, int has_w, SmallVec g, int has_g, long long g_ld,
                                      T* __restrict__ out, int M, int heads, int dv, float eps, float mult,
                                      int gate_silu) {
  pdl_begin();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (long long)M * heads) return;
  const long long m = unit / heads;
  const int h = (int)(unit - m * heads);
  const float* ar = a + unit * a_stride;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) {
    float o = ar[c];
    if (second) o -= lambda * ar[second + c];
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  const float inv = mult / sqrtf(ss / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    float o = ar[c];
    if (second) o -= lambda * ar[second + c];
    const int col = h * dv + c;
    o *= inv;
    if (has_w) o *= w[col];
    if (has_g) {
      const float z = g[(size_t)(m * g_ld + col)];
      o *= gate_silu ? z * sigmoid_f(z) : sigmoid_f(z);
    }
    out[m * (long long)heads * dv + col] = from_f<T>(o);
  }
}

SNK_API int snk_head_norm_gate(const float* a, int a_stride, int second, float lambda, const void* w, int w_f32,
                               const void* g, int g_f32, long long g_ld, void* out, int M, int heads, int dv, float eps,
                               float mult, int gate_silu, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (heads <= 0 || dv <= 0 || a_stride < dv + second) return SNK_ERR_SIZE;
  const long long units = (long long)M * heads;
  const int warps = 8;
  const long long blocks = (units + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return SNK_ERR_SIZE;
  SNK_DISPATCH(dtype, snk_launch(head_norm_gate_kernel<T>, dim3((unsigned)blocks), dim3(warps * 32), 0, stream,
                                 a, a_stride, second, lambda, SmallVec{w, w_f32}, (int)(w != nullptr),
                                 SmallVec{g, g_f32}, (int)(g != nullptr), g_ld, static_cast<T*>(out), M, heads, dv, eps, mult,
                                 gate_silu));
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void act_rows_kernel(const T* __restrict__ x, T* __restrict__ out, long long n, int act) {
  pdl_begin();
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = from_f<T>(act_apply(to_f<T>(x[i]), act));
}

SNK_API int snk_act_rows(const void* x, void* out, long long n, int act, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (act < 0 || act > ACT_RELU2) return SNK_ERR_SIZE;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  SNK_DISPATCH(dtype, snk_launch(act_rows_kernel<T>, dim3(blocks), dim3(256), 0, stream, static_cast<const T*>(x),
                                 static_cast<T*>(out), n, act));
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// One warp per row: out[m, 0:n) = x[m, off + (0:n)] / sqrt(mean(x^2) + eps) * w.
template <typename T>
__global__ void rms_cols_kernel(const T* __restrict__ x, long long ld, int off, SmallVec w, T* __restrict__ out,
                                int M, int n, float eps) {
  pdl_begin();
  const int lane = threadIdx.x & 31;
  const long long m = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= M) return;
  const T* row = x + m * ld + off;
  float ss = 0.f;
  for (int c = lane; c < n; c += 32) {
    const float v = to_f<T>(row[c]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)n + eps);
  for (int c = lane; c < n; c += 32) out[m * n + c] = from_f<T>(to_f<T>(row[c]) * inv * w[c]);
}

SNK_API int snk_rms_cols(const void* x, long long ld, int off, const void* w, int w_f32, void* out, int M, int n,
                         float eps, int dtype, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (n <= 0 || off < 0 || ld < off + n) return SNK_ERR_SIZE;
  const int warps = 4;
  SNK_DISPATCH(dtype, snk_launch(rms_cols_kernel<T>, dim3((M + warps - 1) / warps), dim3(warps * 32), 0, stream,
                                 static_cast<const T*>(x), ld, off, SmallVec{w, w_f32}, static_cast<T*>(out), M, n,
                                 eps));
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// One block per output row.  rows (may be null): the rows to normalise, the residual then stays as it is.
// da, db (may be null): float deltas [M, H].  y, pair_pos, pw, k (k = 0: none): routed experts' outputs
// [pairs, H], where each (row, pick) pair's row lies, and the picks' weights.
template <typename T>
__global__ void add_dyt_kernel(float* __restrict__ residual, const float* __restrict__ da,
                               const float* __restrict__ db, const float* __restrict__ y,
                               const int* __restrict__ pair_pos, const float* __restrict__ pw, int k, SmallVec w,
                               SmallVec b, SmallVec alpha, T* __restrict__ out, const int* __restrict__ rows, int H) {
  pdl_begin();
  const size_t m = rows ? rows[blockIdx.x] : blockIdx.x;
  const float al = alpha[0];
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = residual[m * H + i];
    if (da || db || k) {
      float d = da ? da[m * H + i] : 0.f;
      if (db) d += db[m * H + i];
      if (k) {
        float e = 0.f;
        for (int j = 0; j < k; ++j) e = fmaf(pw[m * k + j], y[(size_t)pair_pos[m * k + j] * H + i], e);
        d += e;
      }
      v += d;
      if (!rows) residual[m * H + i] = v;
    }
    out[(size_t)blockIdx.x * H + i] = from_f<T>(tanhf(al * v) * w[i] + b[i]);
  }
}

SNK_API int snk_add_dyt(float* residual, const float* da, const float* db, const float* y, const int* pair_pos,
                        const float* pw, int k, const void* w, const void* b, const void* alpha, int small_f32,
                        void* out, const int* rows, int R, int H, int dtype, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (H <= 0 || k < 0) return SNK_ERR_SIZE;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  SNK_DISPATCH(dtype, snk_launch(add_dyt_kernel<T>, dim3(R), dim3(threads), 0, stream, residual, da, db, y, pair_pos,
                                 pw, k, SmallVec{w, small_f32}, SmallVec{b, small_f32}, SmallVec{alpha, small_f32},
                                 static_cast<T*>(out), rows, H));
  SNK_LAUNCH_CHECK();
  return 0;
}
