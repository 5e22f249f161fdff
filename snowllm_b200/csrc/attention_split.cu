// Windowed grouped-query attention over a paged cache whose keys and values have widths of their own,
// with what the plain kernel (attention.cu) does not have:
//
//   * keys [page, kv head, page_size, maps*dk] and values [page, kv head, page_size, dv] in two pools;
//   * `maps` softmax maps per head over the same values: q is [M, nq, dk] with nq = heads * maps, query
//     head (h, map) reads the key at offset map*dk of kv head h / group, and every map has an output row
//     of its own [M, nq, dv] (a mixer that subtracts one map from another does so afterwards);
//   * a bias per (query head, distance): s = (q . k) * scale + bias[head][min(i - j, bias_len - 1)];
//   * `window` > 0: the last `window` keys; < 0: the keys of the query's own block of -window positions
//     (blocks counted from position 0); a factor per query head on the scale; a sink per query head (one
//     more term exp(sink) in the softmax's sum, without a key or a value);
//   * `keep` > 0: beside its window a query reaches the positions below `keep` (the sequence's first tokens);
//   * bias_len < 0: `bias` holds one slope per query head and slope * (i - j) is taken off the scaled score;
//   * `gate`: a logit per (row, query head); the head's output is multiplied by its sigmoid;
//   * scores, softmax weights and the products with the values in float whatever the cache dtype (the
//     weights are never rounded to 16 bits), output in float or in the compute dtype.
//
// A block serves up to R consecutive rows of one request and one kv head: its warps take (row, query
// head) units in turns, all reading the same tiles of 32 keys and values from shared memory (16-byte
// cp.async, three tiles in flight; rows that are not 16-byte multiples are copied element by element).
// Tiles are aligned to absolute positions, and a unit walks only the tiles that its own window touches,
// in ascending order: what a row computes depends on its position alone, not on the rows beside it.
//
// The first kernel of the file prepares the step's rows: per-head RMS norm of q and k, rotation of the
// first rot_dim elements of each head (split halves; cos and sin times a magnitude), q out, k and v into
// their pages.
#include "common.cuh"

#define SA_TILE 32
#define SA_STAGES 3

template <typename T> struct SaVec;
template <> struct SaVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
};
template <> struct SaVec<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
  }
};

__device__ __forceinline__ void sa_cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void sa_cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void sa_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}

// ---------------------------------------------------------------------------------------------
// One warp per (row, head) of q, k and v.  proj: the fused projection's output, row pitch ld, with q at
// column q_off ([nq, dk]), k at k_off ([nkh, dk], nkh = kv heads * maps) and v at v_off ([nkv, dv]).
template <typename T>
__global__ void split_prepare_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                                     const float* __restrict__ proj_bias,
                                     SmallVec q_gamma, SmallVec k_gamma, int has_norm, float eps,
                                     const float* __restrict__ inv_freq, int rot_dim, float rot_mult,
                                     const int* __restrict__ positions, const int* __restrict__ row_seg,
                                     const int* __restrict__ block_table, int max_pages, int page_size,
                                     T* __restrict__ kpool, T* __restrict__ vpool, T* __restrict__ q_out,
                                     int nq, int nkh, int nkv, int dk, int dv, int write_kv) {
  pdl_begin();
  extern __shared__ float sp_sh[];                     // [warps][dk]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m = blockIdx.x;
  const int unit = blockIdx.y * (blockDim.x >> 5) + warp;
  const int units = nq + (write_kv ? nkh + nkv : 0);
  if (unit >= units) return;
  const T* row = proj + (size_t)m * ld;
  const int pos = positions[m];
  int page = 0;
  if (unit >= nq) page = block_table[(size_t)row_seg[m] * max_pages + pos / page_size];
  if (unit >= nq + nkh) {                              // a value head: copy
    const int h = unit - nq - nkh;
    const T* src = row + v_off + (size_t)h * dv;
    T* dst = vpool + (((size_t)page * nkv + h) * page_size + pos % page_size) * dv;
    if (proj_bias) {
      const float* bs = proj_bias + v_off + (size_t)h * dv;
      for (int d = lane; d < dv; d += 32) dst[d] = from_f<T>(to_f<T>(src[d]) + bs[d]);
    } else {
      for (int d = lane; d < dv; d += 32) dst[d] = src[d];
    }
    return;
  }
  const bool is_q = unit < nq;
  const int h = is_q ? unit : unit - nq;
  const T* src = row + (is_q ? q_off : k_off) + (size_t)h * dk;
  float* xs = sp_sh + (size_t)warp * dk;
  const float* bs = proj_bias ? proj_bias + (is_q ? q_off : k_off) + (size_t)h * dk : nullptr;
  float ss = 0.f;
  for (int d = lane; d < dk; d += 32) {
    const float v = to_f<T>(src[d]) + (bs ? bs[d] : 0.f);
    xs[d] = v;
    ss = fmaf(v, v, ss);
  }
  if (has_norm == 2) {
    // one root mean square over ALL heads of q (or of k): every warp of the row forms the same sum in the
    // same order; the weight has the projection's size
    const int n = (is_q ? nq : nkh) * dk;
    const T* all = row + (is_q ? q_off : k_off);
    const float* ball = proj_bias ? proj_bias + (is_q ? q_off : k_off) : nullptr;
    float sa = 0.f;
    for (int d = lane; d < n; d += 32) {
      const float v = to_f<T>(all[d]) + (ball ? ball[d] : 0.f);
      sa = fmaf(v, v, sa);
    }
    sa = warp_sum(sa);
    const float inv = 1.f / sqrtf(sa / (float)n + eps);
    const SmallVec& g = is_q ? q_gamma : k_gamma;
    for (int d = lane; d < dk; d += 32) xs[d] = xs[d] * inv * (g.p ? g[(size_t)h * dk + d] : 1.f);
  } else if (has_norm) {
    ss = warp_sum(ss);
    const float inv = 1.f / sqrtf(ss / (float)dk + eps);
    const SmallVec& g = is_q ? q_gamma : k_gamma;
    if (g.p) {
      for (int d = lane; d < dk; d += 32) xs[d] = xs[d] * inv * g[d];
    } else {                                           // a norm without a weight
      for (int d = lane; d < dk; d += 32) xs[d] = xs[d] * inv;
    }
  }
  __syncwarp();
  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)m * nq + h) * dk;
  } else {
    // key head h = kv head * maps + map: the maps of a kv head lie side by side in one row of the pool
    const int maps = nkh / nkv;
    dst = kpool + ((((size_t)page * nkv + h / maps) * page_size + pos % page_size) * maps + h % maps) * dk;
  }
  const int half = rot_dim >> 1;
  for (int d = lane; d < dk; d += 32) {
    float v = xs[d];
    if (d < rot_dim) {
      const int i = d < half ? d : d - half;
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      sn *= rot_mult;
      cs *= rot_mult;
      v = d < half ? xs[d] * cs - xs[d + half] * sn : xs[d] * cs + xs[d - half] * sn;
    }
    dst[d] = from_f<T>(v);
  }
}

// The same for rows of 16-byte vectors: a block takes one row, a thread IT vectors of it (all of their loads in
// flight before the first is used), the lanes of a head sit side by side in a warp (dk / VEC of them, a power of
// two), so that the head's sum of squares and the rotation partner (rot_dim / 2 elements away: a whole number of
// vectors) come by shuffles; the sum over a whole projection goes through the block; the row's sines and cosines
// are worked out once, in shared memory.
template <typename T, int IT>
__global__ void __launch_bounds__(256)
split_prepare_vec_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                         const float* __restrict__ proj_bias, SmallVec q_gamma, SmallVec k_gamma, int has_norm,
                         float eps, const float* __restrict__ inv_freq, int rot_dim, float rot_mult,
                         const int* __restrict__ positions, const int* __restrict__ row_seg,
                         const int* __restrict__ block_table, int max_pages, int page_size,
                         T* __restrict__ kpool, T* __restrict__ vpool, T* __restrict__ q_out,
                         int nq, int nkh, int nkv, int dk, int dv, int write_kv) {
  pdl_begin();
  constexpr int VEC = SaVec<T>::N;
  __shared__ float red[33];
  extern __shared__ float2 sp_tab[];                   // [rot_dim / 2] (cos, sin) of the row's angles
  const int m = blockIdx.x;
  const int lph = dk / VEC, vph = dv / VEC;            // vectors per head of q and k, and of v
  const int nqv = nq * lph, nkv_ = write_kv ? nkh * lph : 0, nvv = write_kv ? nkv * vph : 0;
  const int total = nqv + nkv_ + nvv;
  const T* row = proj + (size_t)m * ld;
  const int pos = positions[m];
  const int half = rot_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    sp_tab[i] = make_float2(cs * rot_mult, sn * rot_mult);
  }
  uint4 raw[IT];
  int col[IT];                                         // the vector's first column in the projection
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    col[it] = -1;
    if (v < total) {
      col[it] = v < nqv ? q_off + v * VEC : (v < nqv + nkv_ ? k_off + (v - nqv) * VEC : v_off + (v - nqv - nkv_) * VEC);
      raw[it] = *reinterpret_cast<const uint4*>(row + col[it]);
    }
  }
  float x[IT][VEC];
  float sq = 0.f, sk = 0.f;                            // this thread's share of the sums over all of q and all of k
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
#pragma unroll
    for (int e = 0; e < VEC; ++e) x[it][e] = 0.f;
    if (col[it] >= 0) {
      SaVec<T>::unpack(raw[it], x[it]);
      if (proj_bias) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[it][e] += proj_bias[col[it] + e];
      }
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss = fmaf(x[it][e], x[it][e], ss);
      if (v < nqv) sq += ss;
      else if (v < nqv + nkv_) sk += ss;
    }
  }
  float inv_q = 1.f, inv_k = 1.f;
  if (has_norm == 2) {
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    inv_q = 1.f / sqrtf(sq / (float)(nq * dk) + eps);
    inv_k = nkv_ ? 1.f / sqrtf(sk / (float)(nkh * dk) + eps) : 1.f;
  } else {
    __syncthreads();                                   // the table of angles is written
  }
  const int lane = threadIdx.x & 31;
  int page = 0;
  if (write_kv) page = block_table[(size_t)row_seg[m] * max_pages + pos / page_size];
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    const bool is_q = v < nqv, is_k = !is_q && v < nqv + nkv_, is_v = !is_q && !is_k && v < total;
    const int hv = is_q ? v : v - nqv;                 // vector within the q (or k) region
    const int h = hv / lph, li = hv - h * lph;         // head, vector of the head
    float inv = 1.f;
    if (has_norm == 1) {                               // a head's own root mean square: every lane takes part
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < VEC; ++e) ss = fmaf(x[it][e], x[it][e], ss);
      for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      inv = 1.f / sqrtf(ss / (float)dk + eps);
    } else if (has_norm == 2) {
      inv = is_q ? inv_q : inv_k;
    }
    if ((is_q || is_k) && has_norm) {
      const SmallVec& g = is_q ? q_gamma : k_gamma;
      const size_t g0 = (has_norm == 2 ? (size_t)h * dk : 0) + (size_t)li * VEC;
#pragma unroll
      for (int e = 0; e < VEC; ++e) x[it][e] = x[it][e] * inv * (g.p ? g[g0 + e] : 1.f);
    }
    if (rot_dim > 0) {                                 // the partner half a rotation away: every lane takes part
      const int d0 = li * VEC, hvn = half / VEC;
      const bool low = d0 < half, turns = (is_q || is_k) && d0 < rot_dim;
      const int src = turns ? (low ? lane + hvn : lane - hvn) : lane;
      float y[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) y[e] = __shfl_sync(0xffffffffu, x[it][e], src);
      if (turns) {
        const int i0 = low ? d0 : d0 - half;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float2 cs = sp_tab[i0 + e];
          x[it][e] = low ? x[it][e] * cs.x - y[e] * cs.y : x[it][e] * cs.x + y[e] * cs.y;
        }
      }
    }
    if (!(is_q || is_k || is_v)) continue;
    T* dst;
    if (is_q) {
      dst = q_out + ((size_t)m * nq + h) * dk + li * VEC;
    } else if (is_k) {
      const int maps = nkh / nkv;
      dst = kpool + ((((size_t)page * nkv + h / maps) * page_size + pos % page_size) * maps + h % maps) * dk + li * VEC;
    } else {
      const int vv = v - nqv - nkv_;
      const int hh = vv / vph, lv = vv - hh * vph;
      dst = vpool + (((size_t)page * nkv + hh) * page_size + pos % page_size) * dv + lv * VEC;
    }
#pragma unroll
    for (int e = 0; e < VEC; e += 4) store4<T>(dst + e, x[it][e], x[it][e + 1], x[it][e + 2], x[it][e + 3]);
  }
}

SNK_API int snk_split_prepare(const void* proj, long long ld, int q_off, int k_off, int v_off,
                              const float* proj_bias, const void* q_gamma,
                              const void* k_gamma, int gamma_f32, int has_norm, float eps, const float* inv_freq,
                              int rot_dim, float rot_mult, const int* positions, const int* row_seg,
                              const int* block_table, int max_pages, int page_size, void* kpool, void* vpool,
                              void* q_out, int M, int nq, int nkh, int nkv, int dk, int dv, int write_kv, int dtype,
                              cudaStream_t stream) {
  if (M <= 0) return 0;
  if (nq <= 0 || dk <= 0 || rot_dim < 0 || rot_dim > dk || (rot_dim & 1)) return SNK_ERR_SIZE;
  if (write_kv && (nkv <= 0 || nkh <= 0 || nkh % nkv || dv <= 0)) return SNK_ERR_SIZE;
  {
    // rows of 16-byte vectors whose heads' lanes fit a warp: the vector kernel
    const int vec = dtype == SNK_F32 ? 4 : 8;
    const size_t esz = dtype == SNK_F32 ? 4 : 2;
    const int lph = dk / vec;
    const int total = (nq * dk + (write_kv ? nkh * dk + nkv * dv : 0)) / vec;
    const bool fits = dk % vec == 0 && lph >= 1 && lph <= 32 && (lph & (lph - 1)) == 0 && (dv % vec == 0 || !write_kv) &&
                      (rot_dim / 2) % vec == 0 && q_off % vec == 0 && (!write_kv || (k_off % vec == 0 && v_off % vec == 0)) &&
                      ld % vec == 0 && (uintptr_t)proj % 16 == 0 && (uintptr_t)q_out % 16 == 0 &&
                      (!write_kv || ((uintptr_t)kpool % 16 == 0 && (uintptr_t)vpool % 16 == 0)) && total <= 256 * 8 &&
                      (rot_dim == 0 || inv_freq != nullptr) && esz * vec == 16;
    if (fits && M <= 2147483647) {
      const int iters = (total + 255) / 256;
      const size_t tab = (size_t)(rot_dim / 2) * sizeof(float2);
#define SP_VEC(I_)                                                                                            \
  snk_launch(split_prepare_vec_kernel<T, I_>, dim3(M), dim3(256), tab, stream, static_cast<const T*>(proj), ld,    \
             q_off, k_off, v_off, proj_bias, SmallVec{q_gamma, gamma_f32}, SmallVec{k_gamma, gamma_f32}, has_norm,  \
             eps, inv_freq, rot_dim, rot_mult, positions, row_seg, block_table, max_pages, page_size,            \
             static_cast<T*>(kpool), static_cast<T*>(vpool), static_cast<T*>(q_out), nq, nkh, nkv, dk, dv, write_kv)
      SNK_DISPATCH(dtype, {
        if (iters <= 1) SP_VEC(1);
        else if (iters <= 2) SP_VEC(2);
        else if (iters <= 4) SP_VEC(4);
        else SP_VEC(8);
      });
#undef SP_VEC
      SNK_LAUNCH_CHECK();
      return 0;
    }
  }
  const int units = nq + (write_kv ? nkh + nkv : 0);
  const int warps = units < 8 ? units : 8;
  dim3 grid(M, (units + warps - 1) / warps);
  const size_t smem = (size_t)warps * dk * sizeof(float);
  if (smem > 48 * 1024) return SNK_ERR_SIZE;
  SNK_DISPATCH(dtype, snk_launch(split_prepare_kernel<T>, dim3(grid), dim3(warps * 32), smem, stream,
                                 static_cast<const T*>(proj), ld, q_off, k_off, v_off, proj_bias,
                                 SmallVec{q_gamma, gamma_f32}, SmallVec{k_gamma, gamma_f32}, has_norm, eps, inv_freq,
                                 rot_dim, rot_mult, positions, row_seg, block_table, max_pages, page_size,
                                 static_cast<T*>(kpool), static_cast<T*>(vpool), static_cast<T*>(q_out), nq, nkh,
                                 nkv, dk, dv, write_kv));
  SNK_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------------------------------
// DPL: output elements per lane (dv <= 32 * DPL); UPW: (row, head) units per warp.
template <typename T, int DPL, int UPW>
__global__ void split_attention_kernel(
    const T* __restrict__ q, const T* __restrict__ kpool, const T* __restrict__ vpool,
    const int* __restrict__ block_table, int max_pages, int page_size, const int* __restrict__ positions,
    const int* __restrict__ row_seg, const int* __restrict__ tiles, void* __restrict__ out, int out_f32,
    int nq, int nkv, int maps, int dk, int dv, int window, float scale, const float* __restrict__ bias,
    int bias_len, const float* __restrict__ head_scale, const float* __restrict__ sink, int keep,
    const T* __restrict__ gate, long long gate_ld, int vec_ok, int chunk,
    int num_chunks, float* __restrict__ part_o, float* __restrict__ part_ml) {
  pdl_begin();
  extern __shared__ __align__(16) unsigned char sa_raw[];
  constexpr int VEC = SaVec<T>::N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int m0 = tiles ? tiles[2 * blockIdx.x] : (int)blockIdx.x;
  const int rows = tiles ? tiles[2 * blockIdx.x + 1] : 1;
  const int kvh = blockIdx.y;
  const int hpv = nq / nkv;                              // query heads (maps counted) per kv head
  const int units = rows * hpv;
  const int pos0 = positions[m0];
  int lo = first_key(pos0, window);
  int hi = pos0 + rows - 1;                              // the last row's own position
  if (num_chunks > 1) {
    // single rows with their keys cut into chunks aligned to absolute positions: this block takes one
    // chunk and leaves (o, max, sum) for the merge (attention.cu), which adds the chunks in order
    int base;
    bool inside;
    if (!chunk_keys(pos0, window, keep, chunk, (int)blockIdx.z, lo, hi, base, inside)) return;
    if (!inside) window = 0;                             // a chunk of kept keys: the row reaches all of it
    keep = 0;
  }
  const int kw = maps * dk;                              // a key row holds the maps side by side

  const int k_bytes = kw * (int)sizeof(T), v_bytes = dv * (int)sizeof(T);
  const int k_stride = ((k_bytes + 15) & ~15) + 16, v_stride = ((v_bytes + 15) & ~15) + 16;
  const int stage_bytes = SA_TILE * (k_stride + v_stride);
  float* qs = reinterpret_cast<float*>(sa_raw + (size_t)SA_STAGES * stage_bytes);

  for (int i = threadIdx.x; i < units * dk; i += blockDim.x) {
    const int u = i / dk, d = i - u * dk;
    const int r = u / hpv, hh = u - r * hpv;
    const float hs = head_scale ? scale * head_scale[kvh * hpv + hh] : scale;
    qs[i] = to_f<T>(q[((size_t)(m0 + r) * nq + kvh * hpv + hh) * dk + d]) * hs;
  }
  const int* bt = block_table + (size_t)row_seg[m0] * max_pages;
  const int t_first = (lo / SA_TILE) * SA_TILE;
  // kept first keys that lie before the walk's first tile come in tiles of their own, ahead of it
  const int nkeep = keep > 0 ? min((keep + SA_TILE - 1) / SA_TILE, t_first / SA_TILE) : 0;
  const int ntiles = nkeep + (hi - t_first) / SA_TILE + 1;
  auto tile_start = [&](int tile) { return tile < nkeep ? tile * SA_TILE : t_first + (tile - nkeep) * SA_TILE; };

  auto issue = [&](int tile) {
    if (tile < ntiles) {
      const int t0 = tile_start(tile);
      unsigned char* ks = sa_raw + (size_t)(tile % SA_STAGES) * stage_bytes;
      unsigned char* vs = ks + SA_TILE * k_stride;
      if (vec_ok) {
        const int kv_ = k_bytes / 16, vv_ = v_bytes / 16, per = kv_ + vv_;
        for (int v = threadIdx.x; v < SA_TILE * per; v += blockDim.x) {
          const int j = v / per, c = v - j * per;
          const int kp = t0 + j;
          const bool valid = kp <= hi && (kp >= lo || kp < keep);
          const T* src = kpool;
          unsigned char* dst = c < kv_ ? ks + j * k_stride + c * 16 : vs + j * v_stride + (c - kv_) * 16;
          if (valid) {
            const size_t slot = ((size_t)bt[kp / page_size] * nkv + kvh) * page_size + kp % page_size;
            src = c < kv_ ? kpool + slot * kw + c * VEC : vpool + slot * dv + (c - kv_) * VEC;
          }
          sa_cp_async16(dst, src, valid);
        }
      } else {
        const int per = kw + dv;
        for (int v = threadIdx.x; v < SA_TILE * per; v += blockDim.x) {
          const int j = v / per, c = v - j * per;
          const int kp = t0 + j;
          T val = from_f<T>(0.f);
          if (kp <= hi && (kp >= lo || kp < keep)) {
            const size_t slot = ((size_t)bt[kp / page_size] * nkv + kvh) * page_size + kp % page_size;
            val = c < kw ? kpool[slot * kw + c] : vpool[slot * dv + (c - kw)];
          }
          if (c < kw) reinterpret_cast<T*>(ks + j * k_stride)[c] = val;
          else reinterpret_cast<T*>(vs + j * v_stride)[c - kw] = val;
        }
      }
    }
    sa_cp_async_commit();
  };

  // a sink is one more term exp(sink) of the row's sum that has no key: the block that holds the row's
  // first keys starts from (maximum = sink, sum = 1)
  const bool sink_here = sink != nullptr && (num_chunks <= 1 || blockIdx.z == 0);
  float mx[UPW], l[UPW], o[UPW][DPL];
#pragma unroll
  for (int i = 0; i < UPW; ++i) {
    const int u0 = warp + nwarps * i;
    mx[i] = -INFINITY;
    l[i] = 0.f;
    if (sink_here && u0 < units) {
      mx[i] = sink[kvh * hpv + u0 % hpv];
      l[i] = 1.f;
    }
#pragma unroll
    for (int e = 0; e < DPL; ++e) o[i][e] = 0.f;
  }

#pragma unroll
  for (int s = 0; s < SA_STAGES - 1; ++s) issue(s);
  for (int tile = 0; tile < ntiles; ++tile) {
    sa_cp_async_wait<SA_STAGES - 2>();
    __syncthreads();                                     // the tile is in (and q, the first time round)
    issue(tile + SA_STAGES - 1);
    const int t0 = tile_start(tile);
    const unsigned char* ks = sa_raw + (size_t)(tile % SA_STAGES) * stage_bytes;
    const unsigned char* vs = ks + SA_TILE * k_stride;
    const int kp = t0 + lane;
#pragma unroll
    for (int i = 0; i < UPW; ++i) {
      const int u = warp + nwarps * i;
      if (u >= units) continue;
      const int r = u / hpv, hh = u - r * hpv;
      const int map = hh % maps;
      const int p = pos0 + r;
      const int klo = max(lo, first_key(p, window));
      const int khi = min(p, hi);
      if (t0 > khi || (t0 + SA_TILE - 1 < klo && t0 >= keep)) continue;  // none of this unit's keys in the tile
      const bool valid = kp <= khi && (kp >= klo || kp < keep);
      const float* qw = qs + (size_t)u * dk;
      float s = 0.f;
      if (vec_ok && dk % VEC == 0) {
        const unsigned char* kr = ks + lane * k_stride + map * dk * (int)sizeof(T);
        for (int cv = 0; cv < dk / VEC; ++cv) {
          float f[VEC];
          SaVec<T>::unpack(*reinterpret_cast<const uint4*>(kr + cv * 16), f);
#pragma unroll
          for (int e = 0; e < VEC; e += 4) {
            const float4 q4 = *reinterpret_cast<const float4*>(qw + cv * VEC + e);
            s = fmaf(q4.x, f[e], s);
            s = fmaf(q4.y, f[e + 1], s);
            s = fmaf(q4.z, f[e + 2], s);
            s = fmaf(q4.w, f[e + 3], s);
          }
        }
      } else {
        const T* kr = reinterpret_cast<const T*>(ks + lane * k_stride) + map * dk;
        for (int d = 0; d < dk; ++d) s = fmaf(qw[d], to_f<T>(kr[d]), s);
      }
      if (bias && valid)
        s = bias_len < 0 ? fmaf(-bias[kvh * hpv + hh], (float)(p - kp), s)
                         : s + bias[(size_t)(kvh * hpv + hh) * bias_len + min(p - kp, bias_len - 1)];
      s = valid ? s : -INFINITY;
      const float m_new = fmaxf(mx[i], warp_max(s));     // finite: the tile holds a key of this unit
      const float corr = expf(mx[i] - m_new);            // 0 the first time
      const float pw = valid ? expf(s - m_new) : 0.f;
      l[i] = l[i] * corr + warp_sum(pw);
      mx[i] = m_new;
#pragma unroll
      for (int e = 0; e < DPL; ++e) o[i][e] *= corr;
      for (int j = 0; j < SA_TILE; ++j) {
        const float pj = __shfl_sync(0xffffffffu, pw, j);
        const T* vr = reinterpret_cast<const T*>(vs + j * v_stride);
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
          const int d = lane + 32 * e;
          if (d < dv) o[i][e] = fmaf(pj, to_f<T>(vr[d]), o[i][e]);
        }
      }
    }
  }
  sa_cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < UPW; ++i) {
    const int u = warp + nwarps * i;
    if (u >= units) continue;
    const int r = u / hpv, hh = u - r * hpv;
    if (num_chunks > 1) {
      const size_t slot = ((size_t)blockIdx.x * nq + kvh * hpv + hh) * num_chunks + blockIdx.z;
#pragma unroll
      for (int e = 0; e < DPL; ++e) {
        const int d = lane + 32 * e;
        if (d < dv) part_o[slot * dv + d] = o[i][e];
      }
      if (lane == 0) {
        part_ml[slot * 2] = mx[i];
        part_ml[slot * 2 + 1] = l[i];
      }
      continue;
    }
    float inv = 1.f / l[i];
    if (gate) inv /= 1.f + expf(-to_f<T>(gate[(size_t)(m0 + r) * gate_ld + kvh * hpv + hh]));
    const size_t at = ((size_t)(m0 + r) * nq + kvh * hpv + hh) * dv;
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
      const int d = lane + 32 * e;
      if (d < dv) {
        if (out_f32) static_cast<float*>(out)[at + d] = o[i][e] * inv;
        else static_cast<T*>(out)[at + d] = from_f<T>(o[i][e] * inv);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// The same attention on the tensor cores (bfloat16 only; dk a multiple of 16 up to 16*DKS, dv a multiple of
// 8 up to 8*DVT, at most 16 query heads per kv head and map).  A warp owns 16 (row, query head) slots of ONE
// map: they are the rows of mma.sync m16n8k16.  S = Q K^T is exact (bfloat16 products, float sums); scale,
// bias, mask and the online softmax work on the float fragments; for O += P V the weights are split into two
// bfloat16 terms, p = hi + lo with lo = bf16(p - hi), and both products are taken, so that P keeps 16
// mantissa bits where one bfloat16 keeps 8; the row sums use the float weights themselves.
// Warp w serves map w % maps; its slot s = (w / maps) * 16 + mma row is (row s / G, head s % G of the kv
// head's G = hpv / maps heads).  All warps of a block read the same key and value tiles.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
// Four 8 x 8 matrices of 16-bit elements from shared memory, lane L giving the address of row L % 8 of matrix
// L / 8.  Plain: a lane gets elements 2 (L % 4), + 1 of row L / 4 of each matrix (the B fragment of keys held
// row by row); .trans: rows 2 (L % 4), + 1 of column L / 4 (the B fragment of values held key by key).
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* row) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* row) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// 2^x by the special-function unit (two units in the last place; 2^-inf = 0)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int DKS, int DVT>
__global__ void split_attention_mma_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ kpool, const bf16* __restrict__ vpool,
    const int* __restrict__ block_table, int max_pages, int page_size, const int* __restrict__ positions,
    const int* __restrict__ row_seg, const int* __restrict__ tiles, void* __restrict__ out, int out_f32,
    int nq, int nkv, int maps, int dk, int dv, int window, float scale, const float* __restrict__ bias,
    int bias_len, const float* __restrict__ head_scale, const float* __restrict__ sink, int keep,
    const bf16* __restrict__ gate, long long gate_ld, int chunk, int num_chunks,
    float* __restrict__ part_o, float* __restrict__ part_ml) {
  pdl_begin();
  extern __shared__ __align__(16) unsigned char sa_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = tiles ? tiles[2 * blockIdx.x] : (int)blockIdx.x;
  const int rows = tiles ? tiles[2 * blockIdx.x + 1] : 1;
  const int kvh = blockIdx.y;
  const int hpv = nq / nkv, G = hpv / maps;
  const int pos0 = positions[m0];
  int lo = first_key(pos0, window);
  int hi = pos0 + rows - 1;
  if (num_chunks > 1) {
    int base;
    bool inside;
    if (!chunk_keys(pos0, window, keep, chunk, (int)blockIdx.z, lo, hi, base, inside)) return;
    if (!inside) window = 0;                               // a chunk of kept keys: the row reaches all of it
    keep = 0;
  }
  const int kw = maps * dk;
  const float scale2 = scale * 1.4426950408889634f;
  const int k_bytes = kw * 2, v_bytes = dv * 2;
  const int k_stride = k_bytes + 16, v_stride = v_bytes + 16;
  const int stage_bytes = SA_TILE * (k_stride + v_stride);

  // this warp's map and its two rows' slots (mma rows lane/4 and lane/4 + 8)
  const int map = warp % maps;
  const int quad = lane >> 2, tq = lane & 3;
  const int slots = rows * G;
  int p_row[2], head[2];
  bool live[2];
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    const int s = (warp / maps) * 16 + quad + 8 * h2;
    live[h2] = s < slots;
    const int r = live[h2] ? s / G : 0;
    p_row[h2] = pos0 + r;
    head[h2] = kvh * hpv + (live[h2] ? (s % G) : 0) * maps + map;
  }
  const bool warp_live = (warp / maps) * 16 < slots;

  // Q fragments straight from global memory: a0 (row A, d 2tq..), a1 (row B), a2 (row A, d + 8), a3 (row B, d + 8)
  uint32_t qa[DKS][4];
#pragma unroll
  for (int ks = 0; ks < DKS; ++ks) {
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      uint32_t x0 = 0, x1 = 0;
      if (live[h2] && ks * 16 < dk) {
        const bf16* qr = q + ((size_t)(m0 + (p_row[h2] - pos0)) * nq + head[h2]) * dk + ks * 16 + tq * 2;
        x0 = *reinterpret_cast<const uint32_t*>(qr);
        x1 = *reinterpret_cast<const uint32_t*>(qr + 8);
      }
      qa[ks][h2] = x0;
      qa[ks][2 + h2] = x1;
    }
  }

  const int* bt = block_table + (size_t)row_seg[m0] * max_pages;
  const int t_first = (lo / SA_TILE) * SA_TILE;
  // kept first keys that lie before the walk's first tile come in tiles of their own, ahead of it
  const int nkeep = keep > 0 ? min((keep + SA_TILE - 1) / SA_TILE, t_first / SA_TILE) : 0;
  const int ntiles = nkeep + (hi - t_first) / SA_TILE + 1;
  auto tile_start = [&](int tile) { return tile < nkeep ? tile * SA_TILE : t_first + (tile - nkeep) * SA_TILE; };
  // which (key of the tile, 16-byte vector of its row) pairs this thread copies: the same for every tile
  const int kv_ = k_bytes / 16, vv_ = v_bytes / 16, per = kv_ + vv_;
  constexpr int COPIES = 6;                                // 32 keys x up to 48 vectors over 32..128 threads
  int cp_j[COPIES], cp_c[COPIES];
  const int n_copies = (SA_TILE * per + (int)blockDim.x - 1) / (int)blockDim.x;
#pragma unroll
  for (int i = 0; i < COPIES; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    cp_j[i] = v < SA_TILE * per ? v / per : -1;
    cp_c[i] = v - (v / per) * per;
  }
  const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
  auto copy_one = [&](unsigned char* ks_, unsigned char* vs_, int t0, int j, int c) {
    const int kp = t0 + j;
    const bool valid = kp <= hi && (kp >= lo || kp < keep);
    const bf16* src = kpool;
    unsigned char* dst = c < kv_ ? ks_ + j * k_stride + c * 16 : vs_ + j * v_stride + (c - kv_) * 16;
    if (valid) {
      const int pg = page_shift >= 0 ? kp >> page_shift : kp / page_size;
      const size_t slot = ((size_t)bt[pg] * nkv + kvh) * page_size + (kp - pg * page_size);
      src = c < kv_ ? kpool + slot * kw + c * 8 : vpool + slot * dv + (c - kv_) * 8;
    }
    sa_cp_async16(dst, src, valid);
  };
  auto issue = [&](int tile) {
    if (tile < ntiles) {
      const int t0 = tile_start(tile);
      unsigned char* ks_ = sa_raw + (size_t)(tile % SA_STAGES) * stage_bytes;
      unsigned char* vs_ = ks_ + SA_TILE * k_stride;
#pragma unroll
      for (int i = 0; i < COPIES; ++i)
        if (cp_j[i] >= 0) copy_one(ks_, vs_, t0, cp_j[i], cp_c[i]);
      for (int i = COPIES; i < n_copies; ++i) {            // few threads and wide rows: the rest the long way
        const int v = threadIdx.x + i * blockDim.x;
        if (v < SA_TILE * per) copy_one(ks_, vs_, t0, v / per, v - (v / per) * per);
      }
    }
    sa_cp_async_commit();
  };

  float mx[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float scale2h[2];
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    scale2h[h2] = head_scale ? scale2 * head_scale[head[h2]] : scale2;
    if (sink != nullptr && live[h2] && (num_chunks <= 1 || blockIdx.z == 0)) {   // the sink: a term without a key
      mx[h2] = sink[head[h2]] * 1.4426950408889634f;
      l[h2] = 1.f;
    }
  }
  float o[DVT][4];
#pragma unroll
  for (int nt = 0; nt < DVT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
  int klo[2], khi[2];
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    klo[h2] = max(lo, first_key(p_row[h2], window));
    khi[h2] = live[h2] ? min(p_row[h2], hi) : -1;           // a slot nobody owns sees no key
  }

#pragma unroll
  for (int s = 0; s < SA_STAGES - 1; ++s) issue(s);
  for (int tile = 0; tile < ntiles; ++tile) {
    sa_cp_async_wait<SA_STAGES - 2>();
    __syncthreads();
    issue(tile + SA_STAGES - 1);
    const int t0 = tile_start(tile);
    // the warp's slots span positions pos0 + first slot / G .. ; skip tiles none of them reaches
    if (!warp_live) continue;
    {
      const int s_lo = (warp / maps) * 16, s_hi = min(slots - 1, s_lo + 15);
      const int p_lo = pos0 + s_lo / G, p_hi = pos0 + s_hi / G;
      const int w_lo = max(lo, first_key(p_lo, window)), w_hi = min(p_hi, hi);
      if (t0 > w_hi || (t0 + SA_TILE - 1 < w_lo && t0 >= keep)) continue;
    }
    const unsigned char* ks_ = sa_raw + (size_t)(tile % SA_STAGES) * stage_bytes;
    const unsigned char* vs_ = ks_ + SA_TILE * k_stride;
    // S = Q K^T: 4 tiles of 8 keys
    float sc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
      // lane L: row L % 8 of the tile's 8 keys, 8 elements from (L / 8) * 8 on: two k-steps per instruction
      const unsigned char* kr = ks_ + (nt * 8 + (lane & 7)) * k_stride + (map * dk + (lane >> 3) * 8) * 2;
#pragma unroll
      for (int kp = 0; kp < DKS / 2; ++kp) {
        if (kp * 32 < dk) {
          uint32_t b[4];
          ldsm_x4(b, kr + kp * 64);
          mma_bf16_16816(sc[nt], qa[2 * kp], b[0], b[1]);
          if (kp * 32 + 16 < dk) mma_bf16_16816(sc[nt], qa[2 * kp + 1], b[2], b[3]);
        }
      }
    }
    // scale, bias, mask; row maxima over the thread's 8 keys, then over the quad
    // (scores and maxima are kept in units of log 2: the weights are 2^(s - m), one instruction each)
    float tmax[2] = {-INFINITY, -INFINITY};
    const bool inner = t0 >= max(klo[0], klo[1]) && t0 + SA_TILE - 1 <= min(khi[0], khi[1]);   // no key is masked
    if (inner) {
      const float* brow[2] = {bias && bias_len > 0 ? bias + (size_t)head[0] * bias_len : nullptr,
                              bias && bias_len > 0 ? bias + (size_t)head[1] * bias_len : nullptr};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h2 = e >> 1;
          float s = sc[nt][e] * scale2h[h2];
          if (bias) {
            const int dist = p_row[h2] - (t0 + nt * 8 + tq * 2 + (e & 1));
            s = bias_len < 0 ? fmaf(-bias[head[h2]] * (float)dist, 1.4426950408889634f, s)
                             : fmaf(brow[h2][min(dist, bias_len - 1)], 1.4426950408889634f, s);
          }
          sc[nt][e] = s;
          tmax[h2] = fmaxf(tmax[h2], s);
        }
      }
    } else {
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h2 = e >> 1;
          const int kp = t0 + nt * 8 + tq * 2 + (e & 1);
          float s = sc[nt][e] * scale2h[h2];
          const bool valid = kp <= khi[h2] && (kp >= klo[h2] || kp < keep);
          if (bias && valid)
            s = bias_len < 0 ? fmaf(-bias[head[h2]] * (float)(p_row[h2] - kp), 1.4426950408889634f, s)
                             : fmaf(bias[(size_t)head[h2] * bias_len + min(p_row[h2] - kp, bias_len - 1)],
                                    1.4426950408889634f, s);
          s = valid ? s : -INFINITY;
          sc[nt][e] = s;
          tmax[h2] = fmaxf(tmax[h2], s);
        }
      }
    }
    float corr[2];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      tmax[h2] = fmaxf(tmax[h2], __shfl_xor_sync(0xffffffffu, tmax[h2], 1));
      tmax[h2] = fmaxf(tmax[h2], __shfl_xor_sync(0xffffffffu, tmax[h2], 2));
      const float m_new = fmaxf(mx[h2], tmax[h2]);
      // a row without a key so far keeps -inf: its weights are 0 and its correction 1
      corr[h2] = m_new == -INFINITY ? 1.f : ex2_approx(mx[h2] - m_new);
      mx[h2] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h2 = e >> 1;
        const float pw = mx[h2] == -INFINITY ? 0.f : ex2_approx(sc[nt][e] - mx[h2]);
        sc[nt][e] = pw;
        psum[h2] += pw;
      }
    }
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      psum[h2] += __shfl_xor_sync(0xffffffffu, psum[h2], 1);
      psum[h2] += __shfl_xor_sync(0xffffffffu, psum[h2], 2);
      l[h2] = l[h2] * corr[h2] + psum[h2];
    }
#pragma unroll
    for (int nt = 0; nt < DVT; ++nt) {
      o[nt][0] *= corr[0]; o[nt][1] *= corr[0];
      o[nt][2] *= corr[1]; o[nt][3] *= corr[1];
    }
    // O += P V in two bfloat16 terms of P; 16 keys per step
#pragma unroll
    for (int kt = 0; kt < 2; ++kt) {
      uint32_t ph[4], pl[4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const float* c = sc[2 * kt + half];
        const float h0 = bf16_round(c[0]), h1 = bf16_round(c[1]), h2_ = bf16_round(c[2]), h3 = bf16_round(c[3]);
        ph[2 * half] = pack_bf16(h0, h1);
        ph[2 * half + 1] = pack_bf16(h2_, h3);
        pl[2 * half] = pack_bf16(c[0] - h0, c[1] - h1);
        pl[2 * half + 1] = pack_bf16(c[2] - h2_, c[3] - h3);
      }
      // lane L: key (L / 8 % 2) * 8 + L % 8 of the step's 16, 8 columns from (L / 16) * 8 on: two column tiles
      // per instruction (a last, odd tile reads the row's pad and is not used)
      const unsigned char* vr = vs_ + (kt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * v_stride + (lane >> 4) * 16;
#pragma unroll
      for (int np = 0; np < DVT / 2; ++np) {
        if (np * 16 < dv) {
          uint32_t b[4];
          ldsm_x4_trans(b, vr + np * 32);
          mma_bf16_16816(o[2 * np], ph, b[0], b[1]);
          mma_bf16_16816(o[2 * np], pl, b[0], b[1]);
          if (np * 16 + 8 < dv) {
            mma_bf16_16816(o[2 * np + 1], ph, b[2], b[3]);
            mma_bf16_16816(o[2 * np + 1], pl, b[2], b[3]);
          }
        }
      }
    }
  }
  sa_cp_async_wait<0>();
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    if (!live[h2]) continue;
    const int r = p_row[h2] - pos0;
    if (num_chunks > 1) {
      const size_t slot = ((size_t)blockIdx.x * nq + head[h2]) * num_chunks + blockIdx.z;
#pragma unroll
      for (int nt = 0; nt < DVT; ++nt) {
        const int d = nt * 8 + tq * 2;
        if (d < dv) {
          part_o[slot * dv + d] = o[nt][2 * h2];
          part_o[slot * dv + d + 1] = o[nt][2 * h2 + 1];
        }
      }
      if (tq == 0) {
        part_ml[slot * 2] = mx[h2] * 0.6931471805599453f;    // the merge works with natural exponents
        part_ml[slot * 2 + 1] = l[h2];
      }
      continue;
    }
    float inv = 1.f / l[h2];
    if (gate) inv /= 1.f + expf(-__bfloat162float(gate[(size_t)(m0 + r) * gate_ld + head[h2]]));
    const size_t at = ((size_t)(m0 + r) * nq + head[h2]) * dv;
#pragma unroll
    for (int nt = 0; nt < DVT; ++nt) {
      const int d = nt * 8 + tq * 2;
      if (d < dv) {
        const float a = o[nt][2 * h2] * inv, b = o[nt][2 * h2 + 1] * inv;
        if (out_f32) {
          static_cast<float*>(out)[at + d] = a;
          static_cast<float*>(out)[at + d + 1] = b;
        } else {
          *reinterpret_cast<uint32_t*>(static_cast<bf16*>(out) + at + d) = pack_bf16(a, b);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Rows that stand alone (decoded tokens) on the tensor cores.  A block takes one row, one kv head and one
// chunk of SD_CHUNK keys at absolute positions; the whole chunk comes into shared memory at once (every copy
// in flight together), then each of the four warps takes 32 of its keys with the kv head's G query heads on
// the rows of the MMA (one map after the other), and the warps' partial (max, sum, o) are merged in warp
// order through shared memory.  More than one chunk: the block leaves its partial for the merge kernel.
#define SD_CHUNK 128
#define SD_WARPS 4

template <int DKS, int DVT>
__global__ void __launch_bounds__(SD_WARPS * 32)
split_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kpool, const bf16* __restrict__ vpool,
                        const int* __restrict__ block_table, int max_pages, int page_size,
                        const int* __restrict__ positions, const int* __restrict__ row_seg,
                        void* __restrict__ out, int out_f32, int nq, int nkv, int maps, int dk, int dv, int window,
                        float scale, const float* __restrict__ bias, int bias_len,
                        const float* __restrict__ head_scale, const float* __restrict__ sink, int keep,
                        const bf16* __restrict__ gate, long long gate_ld, int num_chunks,
                        float* __restrict__ part_o, float* __restrict__ part_ml) {
  pdl_begin();
  extern __shared__ __align__(16) unsigned char sa_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quad = lane >> 2, tq = lane & 3;
  const int m = blockIdx.x, kvh = blockIdx.y;
  const int hpv = nq / nkv, G = hpv / maps;
  const int pos = positions[m];
  int lo, hi, c0;
  bool inside;
  if (!chunk_keys(pos, window, keep, SD_CHUNK, (int)blockIdx.z, lo, hi, c0, inside)) return;
  const int kw = maps * dk;
  const float scale2 = scale * 1.4426950408889634f;
  const int k_bytes = kw * 2, v_bytes = dv * 2;
  const int k_stride = k_bytes + 16, v_stride = v_bytes + 16;
  unsigned char* ks_all = sa_raw;
  unsigned char* vs_all = sa_raw + (size_t)SD_CHUNK * k_stride;
  float* red = reinterpret_cast<float*>(sa_raw + (size_t)SD_CHUNK * (k_stride + v_stride));   // [maps][G][warps][dv + 2]
  const int red_stride = dv + 2;

  {
    const int* bt = block_table + (size_t)row_seg[m] * max_pages;
    const int kv_ = k_bytes / 16, vv_ = v_bytes / 16, per = kv_ + vv_;
    // shifts where the sizes are powers of two (the usual case): the copy loop is then free of divisions
    const int per_shift = (per & (per - 1)) == 0 ? __ffs(per) - 1 : -1;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
    for (int v = threadIdx.x; v < SD_CHUNK * per; v += blockDim.x) {
      const int j = per_shift >= 0 ? v >> per_shift : v / per, c = v - j * per;
      const int kp = c0 + j;
      const bool valid = kp >= lo && kp <= hi;
      const bf16* src = kpool;
      unsigned char* dst = c < kv_ ? ks_all + j * k_stride + c * 16 : vs_all + j * v_stride + (c - kv_) * 16;
      if (valid) {
        const int pg = page_shift >= 0 ? kp >> page_shift : kp / page_size;
        const size_t slot = ((size_t)bt[pg] * nkv + kvh) * page_size + (kp - pg * page_size);
        src = c < kv_ ? kpool + slot * kw + c * 8 : vpool + slot * dv + (c - kv_) * 8;
      }
      sa_cp_async16(dst, src, valid);
    }
    sa_cp_async_commit();
    sa_cp_async_wait<0>();
  }
  __syncthreads();

  const int t0 = c0 + warp * SA_TILE;
  const bool warp_has = t0 <= hi && t0 + SA_TILE - 1 >= lo;
  const unsigned char* ks_ = ks_all + (size_t)warp * SA_TILE * k_stride;
  const unsigned char* vs_ = vs_all + (size_t)warp * SA_TILE * v_stride;
  const bool live[2] = {quad < G, quad + 8 < G};
  for (int map = 0; map < maps; ++map) {
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    float o[DVT][4];
#pragma unroll
    for (int nt = 0; nt < DVT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    if (warp_has) {
      int head[2];
      uint32_t qa[DKS][4];
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) head[h2] = kvh * hpv + (live[h2] ? quad + 8 * h2 : 0) * maps + map;
#pragma unroll
      for (int ks = 0; ks < DKS; ++ks) {
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          uint32_t x0 = 0, x1 = 0;
          if (live[h2] && ks * 16 < dk) {
            const bf16* qr = q + ((size_t)m * nq + head[h2]) * dk + ks * 16 + tq * 2;
            x0 = *reinterpret_cast<const uint32_t*>(qr);
            x1 = *reinterpret_cast<const uint32_t*>(qr + 8);
          }
          qa[ks][h2] = x0;
          qa[ks][2 + h2] = x1;
        }
      }
      float sc[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
        // lane L: row L % 8 of the tile's 8 keys, 8 elements from (L / 8) * 8 on: two k-steps per instruction
        const unsigned char* kr = ks_ + (nt * 8 + (lane & 7)) * k_stride + (map * dk + (lane >> 3) * 8) * 2;
#pragma unroll
        for (int kp = 0; kp < DKS / 2; ++kp) {
          if (kp * 32 < dk) {
            uint32_t b[4];
            ldsm_x4(b, kr + kp * 64);
            mma_bf16_16816(sc[nt], qa[2 * kp], b[0], b[1]);
            if (kp * 32 + 16 < dk) mma_bf16_16816(sc[nt], qa[2 * kp + 1], b[2], b[3]);
          }
        }
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h2 = e >> 1;
          const int kp = t0 + nt * 8 + tq * 2 + (e & 1);
          float sv = sc[nt][e] * (head_scale ? scale2 * head_scale[head[h2]] : scale2);
          const bool valid = live[h2] && kp >= lo && kp <= hi;
          if (bias && valid)
            sv = bias_len < 0 ? fmaf(-bias[head[h2]] * (float)(pos - kp), 1.4426950408889634f, sv)
                              : fmaf(bias[(size_t)head[h2] * bias_len + min(pos - kp, bias_len - 1)],
                                     1.4426950408889634f, sv);
          sv = valid ? sv : -INFINITY;
          sc[nt][e] = sv;
          mrow[h2] = fmaxf(mrow[h2], sv);
        }
      }
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        mrow[h2] = fmaxf(mrow[h2], __shfl_xor_sync(0xffffffffu, mrow[h2], 1));
        mrow[h2] = fmaxf(mrow[h2], __shfl_xor_sync(0xffffffffu, mrow[h2], 2));
      }
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h2 = e >> 1;
          const float pw = mrow[h2] == -INFINITY ? 0.f : ex2_approx(sc[nt][e] - mrow[h2]);
          sc[nt][e] = pw;
          lrow[h2] += pw;
        }
      }
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        lrow[h2] += __shfl_xor_sync(0xffffffffu, lrow[h2], 1);
        lrow[h2] += __shfl_xor_sync(0xffffffffu, lrow[h2], 2);
      }
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
        uint32_t ph[4], pl[4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const float* c = sc[2 * kt + half];
          const float h0 = bf16_round(c[0]), h1 = bf16_round(c[1]), h2_ = bf16_round(c[2]), h3 = bf16_round(c[3]);
          ph[2 * half] = pack_bf16(h0, h1);
          ph[2 * half + 1] = pack_bf16(h2_, h3);
          pl[2 * half] = pack_bf16(c[0] - h0, c[1] - h1);
          pl[2 * half + 1] = pack_bf16(c[2] - h2_, c[3] - h3);
        }
        // lane L: key (L / 8 % 2) * 8 + L % 8 of the step's 16, 8 columns from (L / 16) * 8 on: two column tiles
        // per instruction (a last, odd tile reads the row's pad and is not used)
        const unsigned char* vr = vs_ + (kt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * v_stride + (lane >> 4) * 16;
#pragma unroll
        for (int np = 0; np < DVT / 2; ++np) {
          if (np * 16 < dv) {
            uint32_t b[4];
            ldsm_x4_trans(b, vr + np * 32);
            mma_bf16_16816(o[2 * np], ph, b[0], b[1]);
            mma_bf16_16816(o[2 * np], pl, b[0], b[1]);
            if (np * 16 + 8 < dv) {
              mma_bf16_16816(o[2 * np + 1], ph, b[2], b[3]);
              mma_bf16_16816(o[2 * np + 1], pl, b[2], b[3]);
            }
          }
        }
      }
    }
    // this warp's partial of (map, head) into shared memory: [dv] o, then max and sum
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      if (!live[h2]) continue;
      float* r = red + ((size_t)(map * G + quad + 8 * h2) * SD_WARPS + warp) * red_stride;
#pragma unroll
      for (int nt = 0; nt < DVT; ++nt) {
        const int d = nt * 8 + tq * 2;
        if (d < dv) {
          r[d] = o[nt][2 * h2];
          r[d + 1] = o[nt][2 * h2 + 1];
        }
      }
      if (tq == 0) {
        r[dv] = mrow[h2];
        r[dv + 1] = lrow[h2];
      }
    }
  }
  __syncthreads();
  // the four warps' partials of each (map, head) added in warp order
  for (int i = threadIdx.x; i < hpv * dv; i += blockDim.x) {
    const int mg = i / dv, d = i - mg * dv;              // mg = map * G + head of the kv head
    const float* r = red + (size_t)mg * SD_WARPS * red_stride;
    const int head = kvh * hpv + (mg % G) * maps + mg / G;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w) mx = fmaxf(mx, r[w * red_stride + dv]);
    float l = 0.f, acc = 0.f;
    if (sink != nullptr && blockIdx.z == 0) {            // the sink: one more term of the sum, without a key
      const float sk = sink[head] * 1.4426950408889634f;
      mx = fmaxf(mx, sk);
      l = exp2f(sk - mx);
    }
#pragma unroll
    for (int w = 0; w < SD_WARPS; ++w) {
      const float mw = r[w * red_stride + dv];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - mx);
      l = fmaf(r[w * red_stride + dv + 1], f, l);
      acc = fmaf(r[w * red_stride + d], f, acc);
    }
    if (num_chunks > 1) {
      const size_t slot = ((size_t)m * nq + head) * num_chunks + blockIdx.z;
      part_o[slot * dv + d] = acc;
      if (d == 0) {
        part_ml[slot * 2] = mx * 0.6931471805599453f;
        part_ml[slot * 2 + 1] = l;
      }
    } else {
      float v = acc / l;
      if (gate) v /= 1.f + expf(-__bfloat162float(gate[(size_t)m * gate_ld + head]));
      const size_t at = ((size_t)m * nq + head) * dv + d;
      if (out_f32) static_cast<float*>(out)[at] = v;
      else static_cast<bf16*>(out)[at] = __float2bfloat16_rn(v);
    }
  }
}

// Whether the tensor-core kernel takes these sizes.
static bool sa_mma_ok(int dtype, int nq, int nkv, int maps, int dk, int dv) {
  if (dtype != SNK_BF16 || nkv <= 0 || maps <= 0 || maps > 4 || nq % (nkv * maps)) return false;
  const int G = nq / nkv / maps;
  return G <= 16 && dk % 16 == 0 && dk <= 128 && dv % 8 == 0 && dv <= 128;
}

// Rows of one request that a block serves: the host cuts its tiles to this.  `dk`, `dv`, `dtype`: with sizes
// the tensor-core kernel takes, a block of four warps holds 64 / maps slots per map.  0: sizes nobody takes.
SNK_API int snk_split_attention_tile_rows(int nq, int nkv, int maps, int dk, int dv, int dtype, int decode_only) {
  if (nkv <= 0 || maps <= 0 || nq % (nkv * maps)) return 0;
  const int hpv = nq / nkv;
  if (decode_only) return sa_mma_ok(dtype, nq, nkv, maps, dk, dv) || hpv <= 32 ? 1 : 0;
  if (sa_mma_ok(dtype, nq, nkv, maps, dk, dv)) {
    const int per_map = 16 * (4 / maps), G = hpv / maps;
    return per_map / G;
  }
  return hpv <= 32 ? 32 / hpv : 0;
}

// Keys per chunk for rows that stand alone: SD_CHUNK where the tensor-core kernel serves them, else 256.
SNK_API int snk_split_attention_decode_chunk(int nq, int nkv, int maps, int dk, int dv, int dtype) {
  // Rows of keys and values up to 1,024 bytes together go to the tensor-core kernel.  Measured at 512 bytes a key
  // (two blocks an SM) against the CUDA-core kernel: the same at 64 rows (907 us for four launches over windows of
  // 2,048), faster at 8 rows (a step 0.916 against 0.998 ms); at 256 bytes a key 448 against 634 us.
  static int widest = -1;                                  // SNOWLLM_B200_DECODE_MMA_ROW_BYTES: another bound, for A/B runs
  if (widest < 0) {
    const char* e = getenv("SNOWLLM_B200_DECODE_MMA_ROW_BYTES");
    widest = e ? atoi(e) : 1024;
  }
  return sa_mma_ok(dtype, nq, nkv, maps, dk, dv) && (maps * dk + dv) * 2 <= widest ? SD_CHUNK : 256;
}

// tiles: int32 [num_tiles, 2] = (first row, rows <= tile_rows), consecutive rows of one request; null:
// num_tiles rows, one per block.  num_chunks > 1 (single rows only): each row's keys in chunks of `chunk`
// (a multiple of 32) with partial results in `scratch`, laid out as snk_attention_merge (attention.cu)
// reads them; the caller runs that merge next.
SNK_API int snk_split_attention(const void* q, const void* kpool, const void* vpool, const int* block_table,
                                int max_pages, int page_size, const int* positions, const int* row_seg,
                                const int* tiles, int num_tiles, int tile_rows, void* out, int out_f32, int nq,
                                int nkv, int maps, int dk, int dv, int window, float scale, const float* bias,
                                int bias_len, const float* head_scale, const float* sink, int keep,
                                const void* gate, long long gate_ld, int chunk,
                                int num_chunks, void* scratch, int dtype, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (nkv <= 0 || maps <= 0 || nq % (nkv * maps) || dk <= 0 || dv <= 0 || dv > 256) return SNK_ERR_SIZE;
  const int hpv = nq / nkv;
  if (tile_rows < 1 || nkv > 65535) return SNK_ERR_SIZE;
  if (!tiles) tile_rows = 1;
  if (bias && bias_len == 0) return SNK_ERR_SIZE;
  if (keep < 0 || (keep > 0 && window <= 0)) return SNK_ERR_SIZE;     // kept first keys go with a sliding window
  if (num_chunks < 1 || num_chunks > 65535) return SNK_ERR_SIZE;
  if (num_chunks > 1 && (tiles || scratch == nullptr || chunk <= 0 || chunk % SA_TILE)) return SNK_ERR_SIZE;
  float* part_o = static_cast<float*>(scratch);
  float* part_ml = part_o ? part_o + (size_t)num_tiles * nq * num_chunks * dv : nullptr;
  if (!tiles && chunk == SD_CHUNK && sa_mma_ok(dtype, nq, nkv, maps, dk, dv) && (uintptr_t)kpool % 16 == 0 &&
      (uintptr_t)vpool % 16 == 0 && (uintptr_t)q % 4 == 0) {
    // rows that stand alone, their keys in chunks of SD_CHUNK: the heads of a kv head on the rows of the MMA
    const size_t smem = (size_t)SD_CHUNK * ((size_t)maps * dk * 2 + 16 + (size_t)dv * 2 + 16) +
                        (size_t)hpv * SD_WARPS * (dv + 2) * sizeof(float);
    if (smem > 227 * 1024) return SNK_ERR_SIZE;
    dim3 grid(num_tiles, nkv, num_chunks);
#define SD_MMA(DKS_, DVT_)                                                                                   \
  do {                                                                                                       \
    if (smem > 48 * 1024)                                                                                    \
      cudaFuncSetAttribute(split_decode_mma_kernel<DKS_, DVT_>,                                              \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                          \
    snk_launch(split_decode_mma_kernel<DKS_, DVT_>, dim3(grid), dim3(SD_WARPS * 32), smem, stream,           \
               static_cast<const bf16*>(q), static_cast<const bf16*>(kpool), static_cast<const bf16*>(vpool), \
               block_table, max_pages, page_size, positions, row_seg, out, out_f32, nq, nkv, maps, dk, dv,   \
               window, scale, bias, bias_len, head_scale, sink, keep, static_cast<const bf16*>(gate), gate_ld,   \
               num_chunks, part_o, part_ml);                                                                 \
  } while (0)
    if (dk <= 64 && dv <= 64) SD_MMA(4, 8);
    else if (dk <= 64) SD_MMA(4, 16);
    else if (dv <= 64) SD_MMA(8, 8);
    else SD_MMA(8, 16);
#undef SD_MMA
    SNK_LAUNCH_CHECK();
    return 0;
  }
  if (tiles && sa_mma_ok(dtype, nq, nkv, maps, dk, dv) && (uintptr_t)kpool % 16 == 0 &&
      (uintptr_t)vpool % 16 == 0 && (uintptr_t)q % 4 == 0) {
    const int G = hpv / maps;
    const int slots = tile_rows * G;                       // per map
    if (slots > 16 * (4 / maps)) return SNK_ERR_SIZE;
    const int warps = maps * ((slots + 15) / 16);
    const size_t stage = (size_t)SA_TILE * ((size_t)maps * dk * 2 + 16 + (size_t)dv * 2 + 16);
    const size_t smem = SA_STAGES * stage;
    if (smem > 227 * 1024) return SNK_ERR_SIZE;
    dim3 grid(num_tiles, nkv, num_chunks);
#define SA_MMA(DKS_, DVT_)                                                                                   \
  do {                                                                                                       \
    if (smem > 48 * 1024)                                                                                    \
      cudaFuncSetAttribute(split_attention_mma_kernel<DKS_, DVT_>,                                           \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                          \
    snk_launch(split_attention_mma_kernel<DKS_, DVT_>, dim3(grid), dim3(warps * 32), smem, stream,           \
               static_cast<const bf16*>(q), static_cast<const bf16*>(kpool), static_cast<const bf16*>(vpool), \
               block_table, max_pages, page_size, positions, row_seg, tiles, out, out_f32, nq, nkv, maps,    \
               dk, dv, window, scale, bias, bias_len, head_scale, sink, keep, static_cast<const bf16*>(gate),    \
               gate_ld, chunk, num_chunks, part_o, part_ml);                                                 \
  } while (0)
    if (dk <= 64 && dv <= 64) SA_MMA(4, 8);
    else if (dk <= 64) SA_MMA(4, 16);
    else if (dv <= 64) SA_MMA(8, 8);
    else SA_MMA(8, 16);
#undef SA_MMA
    SNK_LAUNCH_CHECK();
    return 0;
  }
  if (hpv > 32 || tile_rows * hpv > 32) return SNK_ERR_SIZE;
  const int esz = dtype == SNK_F32 ? 4 : 2;
  const int kw = maps * dk;
  const int vec_ok = (kw * esz) % 16 == 0 && (dv * esz) % 16 == 0 && (uintptr_t)kpool % 16 == 0 &&
                     (uintptr_t)vpool % 16 == 0;
  const int cap = tile_rows * hpv;                       // units a block may have to serve
  const int upw = cap > 16 ? 4 : 1;
  const int warps = upw == 1 ? cap : 8;
  const size_t stage = (size_t)SA_TILE * ((((size_t)kw * esz + 15) & ~(size_t)15) + 16 + (((size_t)dv * esz + 15) & ~(size_t)15) + 16);
  const size_t smem = SA_STAGES * stage + (size_t)cap * dk * sizeof(float);
  if (smem > 227 * 1024) return SNK_ERR_SIZE;
  dim3 grid(num_tiles, nkv, num_chunks);
#define SA_LAUNCH(DPL_, UPW_)                                                                          \
  do {                                                                                                 \
    if (smem > 48 * 1024)                                                                              \
      cudaFuncSetAttribute(split_attention_kernel<T, DPL_, UPW_>,                                      \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                    \
    snk_launch(split_attention_kernel<T, DPL_, UPW_>, dim3(grid), dim3(warps * 32), smem, stream,      \
               static_cast<const T*>(q), static_cast<const T*>(kpool), static_cast<const T*>(vpool),   \
               block_table, max_pages, page_size, positions, row_seg, tiles, out, out_f32, nq, nkv,    \
               maps, dk, dv, window, scale, bias, bias_len, head_scale, sink, keep,                    \
               static_cast<const T*>(gate), gate_ld, vec_ok, chunk, num_chunks, part_o, part_ml);      \
  } while (0)
#define SA_LAUNCH_U(DPL_)                  \
  do {                                     \
    if (upw == 1) SA_LAUNCH(DPL_, 1);      \
    else SA_LAUNCH(DPL_, 4);               \
  } while (0)
  SNK_DISPATCH(dtype, {
    if (dv <= 32) SA_LAUNCH_U(1);
    else if (dv <= 64) SA_LAUNCH_U(2);
    else if (dv <= 128) SA_LAUNCH_U(4);
    else SA_LAUNCH_U(8);
  });
#undef SA_LAUNCH_U
#undef SA_LAUNCH
  SNK_LAUNCH_CHECK();
  return 0;
}
