// A residual stream kept as several streams (hyper-connections), and the norm that reads them.
//
//   streams_norm:   X [M, S, W] float.  A sublayer reads u = sum_s in[s] X[s] through its norm and
//                   leaves y; the streams then become, all at once from the old ones,
//                   X'[t] = sum_s mix[s][t] X[s] + out[t] y.  This kernel is the seam between two
//                   sublayers: it applies the update that the sublayer before left pending (y may be a
//                   float tensor, a second one, and routed experts' outputs still in pieces), stores X',
//                   forms the next u and normalises it: the width in `groups` equal consecutive parts,
//                   each over its own sqrt(mean(part^2) + eps), the whole times w.  With `init` the
//                   streams are first set to S copies of a plain residual row.  With `rows` only those
//                   rows come out and the streams stay as they are (the model's last norm on the rows
//                   whose logits are wanted).  S = 1 with mix = out = in = 1 is the plain residual sum
//                   followed by the grouped norm.
//   pair_norm_mix:  out = ca * a / rms(a) * wa + cb * b / rms(b) * wb over the width: two mixers side by
//                   side, each output normalised with a weight of its own.
//
// Sums, statistics and the streams are float; the normalised row is rounded to the compute dtype once.
#include "common.cuh"

#define SN_MAX_STREAMS 8

// VEC consecutive floats of one row (VEC 4: one 16-byte access)
template <int VEC>
__device__ __forceinline__ void sn_load(const float* __restrict__ p, float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    v[0] = *p;
  }
}
template <int VEC>
__device__ __forceinline__ void sn_store(float* __restrict__ p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  else *p = v[0];
}
template <typename T, int VEC>
__device__ __forceinline__ void sn_store_out(T* __restrict__ p, const float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    __align__(16) T t[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) t[e] = from_f<T>(v[e]);
    if constexpr (sizeof(T) == 2) *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(t);
    else *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(t);
  } else {
    *p = from_f<T>(v[0]);
  }
}

#define SN_MAX_PIECES 16       // experts' pieces per row whose places and weights are kept in shared memory

// SMAX: the streams the registers hold (S <= SMAX).  VEC: floats per access (4 needs W and W / groups to be
// multiples of 4 and 16-byte aligned operands).
template <typename T, int SMAX, int VEC>
// (The bound of 768 threads is there for its register limit, 85: three blocks of 256 then share an SM.)
__global__ void __launch_bounds__(SMAX <= 4 ? 768 : 256)
streams_norm_kernel(float* __restrict__ X, const float* __restrict__ init,
                                    const float* __restrict__ da, const float* __restrict__ db,
                                    const float* __restrict__ y, const int* __restrict__ pair_pos,
                                    const float* __restrict__ pw, int k, const float* __restrict__ mix,
                                    const float* __restrict__ outw, const float* __restrict__ inw, SmallVec w,
                                    int groups, float eps, T* __restrict__ out, const int* __restrict__ rows,
                                    int S, int W, int has_update) {
  pdl_begin();
  extern __shared__ __align__(16) float sn_sh[];         // [W] u, then [groups] 1 / rms
  __shared__ int piece_at[SN_MAX_PIECES];
  __shared__ float piece_w[SN_MAX_PIECES];
  float* us = sn_sh;
  float* inv = sn_sh + ((W + 3) & ~3);
  const size_t m = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = X + m * S * W;
  // the stream weights lie in shared memory (every thread reads the same word): in registers they cost a
  // third of the threads an SM could hold, and this kernel lives on loads in flight
  __shared__ float cm[SMAX][SMAX], co[SMAX], ci[SMAX];
  if (threadIdx.x < SMAX * SMAX) {
    const int s = threadIdx.x / SMAX, t = threadIdx.x % SMAX;
    cm[s][t] = (has_update && s < S && t < S) ? mix[s * S + t] : 0.f;
    if (t == 0) {
      co[s] = (has_update && s < S) ? outw[s] : 0.f;
      ci[s] = s < S ? (inw ? inw[s] : 1.f) : 0.f;
    }
  }
  const bool pieces_shared = has_update && k > 0 && k <= SN_MAX_PIECES;
  if (pieces_shared && threadIdx.x >= 64 && threadIdx.x < 64 + k) {
    piece_at[threadIdx.x - 64] = pair_pos[m * k + threadIdx.x - 64];
    piece_w[threadIdx.x - 64] = pw[m * k + threadIdx.x - 64];
  }
  __syncthreads();
  for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
    float x[SMAX][VEC];
    if (init) {
      float v[VEC];
      sn_load<VEC>(init + m * W + i, v);
#pragma unroll
      for (int s = 0; s < SMAX; ++s)
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[s][e] = v[e];
    } else {
#pragma unroll
      for (int s = 0; s < SMAX; ++s) {
        if (s < S) {
          sn_load<VEC>(xr + (size_t)s * W + i, x[s]);
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) x[s][e] = 0.f;
        }
      }
    }
    float u[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) u[e] = 0.f;
    if (has_update) {
      float d[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) d[e] = 0.f;
      if (da) sn_load<VEC>(da + m * W + i, d);
      if (db) {
        float t[VEC];
        sn_load<VEC>(db + m * W + i, t);
#pragma unroll
        for (int e = 0; e < VEC; ++e) d[e] += t[e];
      }
      if (k) {
        float acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
        for (int j = 0; j < k; ++j) {
          const int at = pieces_shared ? piece_at[j] : pair_pos[m * k + j];
          const float wt = pieces_shared ? piece_w[j] : pw[m * k + j];
          float t[VEC];
          sn_load<VEC>(y + (size_t)at * W + i, t);
#pragma unroll
          for (int e = 0; e < VEC; ++e) acc[e] = fmaf(wt, t[e], acc[e]);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) d[e] += acc[e];
      }
#pragma unroll
      for (int t = 0; t < SMAX; ++t) {
        if (t < S) {
          float v[VEC];
#pragma unroll
          for (int e = 0; e < VEC; ++e) {
            v[e] = 0.f;
#pragma unroll
            for (int s = 0; s < SMAX; ++s) v[e] = fmaf(cm[s][t], x[s][e], v[e]);
            v[e] = fmaf(co[t], d[e], v[e]);
            u[e] = fmaf(ci[t], v[e], u[e]);
          }
          if (!rows) sn_store<VEC>(xr + (size_t)t * W + i, v);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < SMAX; ++t) {
        if (t < S) {
          if (init && !rows) sn_store<VEC>(xr + (size_t)t * W + i, x[t]);
#pragma unroll
          for (int e = 0; e < VEC; ++e) u[e] = fmaf(ci[t], x[t][e], u[e]);
        }
      }
    }
    sn_store<VEC>(us + i, u);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int part = W / groups;
  for (int g = warp; g < groups; g += nwarps) {
    float ss = 0.f;
    if constexpr (VEC == 4) {
      for (int i = lane * 4; i < part; i += 128) {
        const float4 v = *reinterpret_cast<const float4*>(us + g * part + i);
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
      }
    } else {
      for (int i = lane; i < part; i += 32) {
        const float v = us[g * part + i];
        ss = fmaf(v, v, ss);
      }
    }
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.f / sqrtf(ss / (float)part + eps);
  }
  __syncthreads();
  for (int i = threadIdx.x * VEC; i < W; i += blockDim.x * VEC) {
    const float scale = inv[i / part];                   // VEC 4: part is a multiple of 4, one group
    float v[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = us[i + e] * scale * w[i + e];
    sn_store_out<T, VEC>(out + (size_t)blockIdx.x * W + i, v);
  }
}

// X: float [M, S, W].  init (may be null): float [M, W].  Pending update (has_update): da, db float [M, W]
// (may be null), y / pair_pos / pw / k the experts' pieces (k = 0: none), mix float [S, S] indexed
// [from, to], outw float [S].  inw: float [S], null for the plain sum.  w: [W] norm weight.  rows (may be
// null): int32 [R].  out: [R, W] in the compute dtype.
SNK_API int snk_streams_norm(float* X, const float* init, const float* da, const float* db, const float* y,
                             const int* pair_pos, const float* pw, int k, const float* mix, const float* outw,
                             const float* inw, const void* w, int w_f32, int groups, float eps, void* out,
                             const int* rows, int R, int S, int W, int has_update, int dtype,
                             cudaStream_t stream) {
  if (R <= 0) return 0;
  if (S <= 0 || S > SN_MAX_STREAMS || W <= 0 || groups <= 0 || W % groups || k < 0) return SNK_ERR_SIZE;
  if (has_update && (!mix || !outw)) return SNK_ERR_SIZE;
  const size_t smem = (size_t)(((W + 3) & ~3) + groups) * sizeof(float);
  if (smem > 200 * 1024) return SNK_ERR_SIZE;
  const uintptr_t all = (uintptr_t)X | (uintptr_t)init | (uintptr_t)da | (uintptr_t)db | (uintptr_t)y | (uintptr_t)out;
  const bool vec = W % 4 == 0 && (W / groups) % 4 == 0 && (all & 15) == 0;
  const int cols = vec ? W / 4 : W;
  // Many rows: blocks of 256 threads, of which an SM holds three (four streams in registers) in different
  // phases, kept its loads in flight better than one block of 512 (a 2,048-row seam 63 -> 43 us).  Few rows:
  // every block has an SM to itself and the widest one is through soonest.  At least 64 + SN_MAX_PIECES
  // threads, and SMAX^2.
  const int threads = cols >= 512 && R < 592 && S <= 4 ? 512 : (cols >= 256 ? 256 : 128);
#define SN_LAUNCH(SMAX_, VEC_)                                                                                \
  do {                                                                                                        \
    auto kernel = streams_norm_kernel<T, SMAX_, VEC_>;                                                        \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    snk_launch(kernel, dim3(R), dim3(threads), smem, stream, X, init, da, db, y, pair_pos, pw, k, mix, outw,  \
               inw, SmallVec{w, w_f32}, groups, eps, static_cast<T*>(out), rows, S, W, has_update);           \
  } while (0)
  SNK_DISPATCH(dtype, {
    if (vec) {
      if (S == 1) SN_LAUNCH(1, 4);
      else if (S <= 2) SN_LAUNCH(2, 4);
      else if (S <= 4) SN_LAUNCH(4, 4);
      else SN_LAUNCH(8, 4);
    } else {
      if (S == 1) SN_LAUNCH(1, 1);
      else if (S <= 2) SN_LAUNCH(2, 1);
      else if (S <= 4) SN_LAUNCH(4, 1);
      else SN_LAUNCH(8, 1);
    }
  });
#undef SN_LAUNCH
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// One block per row; both rows are kept in shared memory between the two passes.
__global__ void pair_norm_mix_kernel(const float* __restrict__ a, const float* __restrict__ b, SmallVec wa,
                                     SmallVec wb, float ca, float cb, float eps, float* __restrict__ out, int W) {
  pdl_begin();
  extern __shared__ __align__(16) float pm_sh[];         // [W] a, [W] b, 33 for the reductions
  float* as = pm_sh;
  float* bs = pm_sh + ((W + 3) & ~3);
  float* red = bs + ((W + 3) & ~3);
  const size_t m = blockIdx.x;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float x = a[m * W + i], z = b[m * W + i];
    as[i] = x;
    bs[i] = z;
    sa = fmaf(x, x, sa);
    sb = fmaf(z, z, sb);
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ia = ca / sqrtf(sa / (float)W + eps), ib = cb / sqrtf(sb / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out[m * W + i] = as[i] * ia * wa[i] + bs[i] * ib * wb[i];
}

SNK_API int snk_pair_norm_mix(const float* a, const float* b, const void* wa, const void* wb, int w_f32, float ca,
                              float cb, float eps, float* out, int M, int W, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (W <= 0) return SNK_ERR_SIZE;
  const size_t smem = (size_t)(2 * ((W + 3) & ~3) + 33) * sizeof(float);
  if (smem > 200 * 1024) return SNK_ERR_SIZE;
  const int threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(pair_norm_mix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  snk_launch(pair_norm_mix_kernel, dim3(M), dim3(threads), smem, stream, a, b, SmallVec{wa, w_f32},
             SmallVec{wb, w_f32}, ca, cb, eps, out, W);
  SNK_LAUNCH_CHECK();
  return 0;
}
