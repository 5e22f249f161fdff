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

template <typename T>
__global__ void streams_norm_kernel(float* __restrict__ X, const float* __restrict__ init,
                                    const float* __restrict__ da, const float* __restrict__ db,
                                    const float* __restrict__ y, const int* __restrict__ pair_pos,
                                    const float* __restrict__ pw, int k, const float* __restrict__ mix,
                                    const float* __restrict__ outw, const float* __restrict__ inw, SmallVec w,
                                    int groups, float eps, T* __restrict__ out, const int* __restrict__ rows,
                                    int S, int W, int has_update) {
  pdl_begin();
  extern __shared__ __align__(16) float sn_sh[];         // [W] u, then [groups] 1 / rms
  float* us = sn_sh;
  float* inv = sn_sh + ((W + 3) & ~3);
  const size_t m = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = X + m * S * W;
  float cm[SN_MAX_STREAMS][SN_MAX_STREAMS], co[SN_MAX_STREAMS], ci[SN_MAX_STREAMS];
#pragma unroll
  for (int s = 0; s < SN_MAX_STREAMS; ++s) {
    co[s] = (has_update && s < S) ? outw[s] : 0.f;
    ci[s] = s < S ? (inw ? inw[s] : 1.f) : 0.f;
#pragma unroll
    for (int t = 0; t < SN_MAX_STREAMS; ++t) cm[s][t] = (has_update && s < S && t < S) ? mix[s * S + t] : 0.f;
  }
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float x[SN_MAX_STREAMS];
    if (init) {
      const float v = init[m * W + i];
#pragma unroll
      for (int s = 0; s < SN_MAX_STREAMS; ++s) x[s] = v;
    } else {
#pragma unroll
      for (int s = 0; s < SN_MAX_STREAMS; ++s) x[s] = s < S ? xr[(size_t)s * W + i] : 0.f;
    }
    float u = 0.f;
    if (has_update) {
      float d = da ? da[m * W + i] : 0.f;
      if (db) d += db[m * W + i];
      if (k) {
        float e = 0.f;
        for (int j = 0; j < k; ++j) e = fmaf(pw[m * k + j], y[(size_t)pair_pos[m * k + j] * W + i], e);
        d += e;
      }
#pragma unroll
      for (int t = 0; t < SN_MAX_STREAMS; ++t) {
        if (t < S) {
          float v = 0.f;
#pragma unroll
          for (int s = 0; s < SN_MAX_STREAMS; ++s) v = fmaf(cm[s][t], x[s], v);
          v = fmaf(co[t], d, v);
          if (!rows) xr[(size_t)t * W + i] = v;
          u = fmaf(ci[t], v, u);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < SN_MAX_STREAMS; ++t) {
        if (t < S) {
          if (init && !rows) xr[(size_t)t * W + i] = x[t];
          u = fmaf(ci[t], x[t], u);
        }
      }
    }
    us[i] = u;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int part = W / groups;
  for (int g = warp; g < groups; g += nwarps) {
    float ss = 0.f;
    for (int i = lane; i < part; i += 32) {
      const float v = us[g * part + i];
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.f / sqrtf(ss / (float)part + eps);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out[(size_t)blockIdx.x * W + i] = from_f<T>(us[i] * inv[i / part] * w[i]);
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
  const int threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
  SNK_DISPATCH(dtype, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(streams_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    snk_launch(streams_norm_kernel<T>, dim3(R), dim3(threads), smem, stream, X, init, da, db, y, pair_pos, pw, k,
               mix, outw, inw, SmallVec{w, w_f32}, groups, eps, static_cast<T*>(out), rows, S, W, has_update);
  });
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
