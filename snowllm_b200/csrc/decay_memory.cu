// Linear attention as a decayed matrix memory, token by token, over a flat batch of segments.
//
// Per head a float matrix S [dk, dv], zero for a fresh request, kept in the request's state slot
// between steps:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t
//
// a_t (the decay of S's rows) and k_t come in one of two forms:
//
//   gated  (HGRN2):     f = low + (1 - low) * sigmoid(z + b) per head and channel, from the projection
//                       z, a bias b and a lower bound `low`;  a_t = f, k_t = 1 - f: what the gate forgets
//                       is what is written.  q = silu(projection).
//   fixed  (retention): a_t = decay[head] for every row; q and k are projections whose first rot_dim
//                       elements per head turn with the position (split halves, angle = position *
//                       inv_freq in float), k times k_scale after the rotation.
//
// The projections arrive as float rows `proj` [M, ld] (q at q_off, k or z at k_off, both [H, dk]; v at
// v_off [H, dv]).  Gates, decays, angles, state and sums are float whatever the model's compute dtype.
//
// A block serves one (segment, head, 32 columns of S).  Eight neighbouring threads share a column: each
// holds an eighth of its rows in registers over the whole segment, and three shuffles add their parts of
// S^T q.  The block meets only to bring the next 32 tokens' q, k and decays into shared memory (gates,
// activations and rotations are evaluated there, off the token loop's chain of dependent instructions).
// The output is the raw o in float [M, H*dv]; per-head norms, weights and gates follow in
// head_norm_gate (sublayer.cu).
//
// A long prompt portion would leave one block per (head, 32 columns) walking thousands of tokens while most
// SMs idle.  The host then cuts every segment into pieces of consecutive rows (`pieces`: int32 [n, 4] =
// segment, first row, rows, flags; bit 0 the segment's first piece, bit 1 its last) and three launches
// replace the one:
//
//   collect  every piece but a segment's last walks its tokens from S = 0 and leaves its own sum L_p and
//            the product D_p of its decays per row in `work` / `work_decay`;
//   scan     per segment, piece after piece: S_(p+1) = diag(D_p) S_p + L_p, starting from the slot's state
//            (zero for a fresh request); S_p takes L_p's place in `work`;
//   emit     every piece walks its tokens again from S_p and writes o; a segment's last piece leaves the
//            state in the slot.
//
// The recurrence is linear in S, so this is the same sum in another order, every term still a float.
#include "common.cuh"

#define DM_CHUNK 32            // tokens brought in at a time
#define DM_COLS 32             // columns of S per block
#define DM_TPC 8               // threads per column

enum { DM_GATED = 0, DM_FIXED = 1 };

enum { DM_WHOLE = 0, DM_COLLECT = 1, DM_EMIT = 2 };
enum { DM_FIRST = 1, DM_LAST = 2 };

template <int DKR, int PHASE>
__global__ void __launch_bounds__(DM_TPC * DM_COLS)
decay_memory_kernel(const float* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, int mode,
                    SmallVec gate_bias, SmallVec gate_low, const float* __restrict__ decay,
                    const float* __restrict__ inv_freq, int rot_dim, float k_scale,
                    const int* __restrict__ positions, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                    float* __restrict__ state, float* __restrict__ out, int H, int dk, int dv,
                    const int4* __restrict__ pieces, float* __restrict__ work, float* __restrict__ work_decay) {
  pdl_begin();
  extern __shared__ __align__(16) float dm_sh[];
  constexpr int RPT = DKR / DM_TPC;                      // rows of S per thread
  int4 piece = make_int4(blockIdx.x, 0, 0, DM_FIRST | DM_LAST);
  if (PHASE != DM_WHOLE) {
    piece = pieces[blockIdx.x];
    if (PHASE == DM_COLLECT && (piece.w & DM_LAST)) return;
  }
  const int b = piece.x, h = blockIdx.y;
  const int sub = threadIdx.x & (DM_TPC - 1);            // which share of the column's rows
  const int c = blockIdx.z * DM_COLS + threadIdx.x / DM_TPC;
  const bool has_col = c < dv;
  const int dkp = (dk + 4 * DM_TPC - 1) / (4 * DM_TPC) * (4 * DM_TPC);
  float* qs = dm_sh;                                     // [DM_CHUNK][dkp]
  float* ks = qs + DM_CHUNK * dkp;                       // [DM_CHUNK][dkp]
  float* as = ks + DM_CHUNK * dkp;                       // [DM_CHUNK][dkp]  decay of each row of S
  float* vs = as + DM_CHUNK * dkp;                       // [DM_CHUNK][DM_COLS]

  const int row0 = PHASE == DM_WHOLE ? cu_seqlens[b] : piece.y;
  const int row1 = PHASE == DM_WHOLE ? cu_seqlens[b + 1] : piece.y + piece.z;
  // where S comes from (null: zero) and where it goes (null: nowhere)
  float* slot = state + ((size_t)seg_slot[b] * H + h) * dk * dv;
  float* mine = PHASE == DM_WHOLE ? nullptr : work + ((size_t)blockIdx.x * H + h) * dk * dv;
  // (a segment's first piece of several reads what the scan left, not the slot that its last piece writes)
  const float* from = PHASE == DM_COLLECT ? nullptr
                    : (piece.w & (DM_FIRST | DM_LAST)) == (DM_FIRST | DM_LAST) ? (seg_start[b] == 0 ? nullptr : slot)
                    : mine;
  float* to = PHASE == DM_COLLECT ? mine : (piece.w & DM_LAST) ? slot : nullptr;

  // register i*4 + e holds row 4 DM_TPC i + 4 sub + e
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT / 4; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = 4 * DM_TPC * i + 4 * sub + e;
      S[i * 4 + e] = (from && has_col && r < dk) ? from[(size_t)r * dv + c] : 0.f;
    }
  float D[PHASE == DM_COLLECT ? RPT : 1];                // the product of each row's decays over the piece
  if (PHASE == DM_COLLECT)
#pragma unroll
    for (int i = 0; i < RPT; ++i) D[i] = 1.f;
  const int col0 = blockIdx.z * DM_COLS;
  const int half = rot_dim >> 1;
  const float head_decay = mode == DM_FIXED ? decay[h] : 0.f;

  for (int t0 = row0; t0 < row1; t0 += DM_CHUNK) {
    const int nt = min(DM_CHUNK, row1 - t0);
    __syncthreads();                                     // everyone is done with the previous chunk
    for (int i = threadIdx.x; i < nt * dkp; i += blockDim.x) {
      const int t = i / dkp, r = i - t * dkp;
      float qv = 0.f, kv = 0.f, av = 0.f;
      if (r < dk) {
        const float* pr = proj + (size_t)(t0 + t) * ld;
        const float* pq = pr + q_off + h * dk;
        const float* pk = pr + k_off + h * dk;
        if (mode == DM_GATED) {
          const float z = pq[r];
          qv = z / (1.f + expf(-z));
          const float low = gate_low[h * dk + r];
          const float f = low + (1.f - low) / (1.f + expf(-(pk[r] + gate_bias[h * dk + r])));
          av = f;
          kv = 1.f - f;
        } else {
          qv = pq[r];
          kv = pk[r];
          if (r < rot_dim) {
            const int j = r < half ? r : r - half;
            float sn, cs;
            sincosf((float)positions[t0 + t] * inv_freq[j], &sn, &cs);
            if (r < half) {
              qv = pq[r] * cs - pq[r + half] * sn;
              kv = pk[r] * cs - pk[r + half] * sn;
            } else {
              qv = pq[r] * cs + pq[r - half] * sn;
              kv = pk[r] * cs + pk[r - half] * sn;
            }
          }
          kv *= k_scale;
          av = head_decay;
        }
      }
      qs[i] = qv;
      ks[i] = kv;
      as[i] = av;
    }
    for (int i = threadIdx.x; i < nt * DM_COLS; i += blockDim.x) {
      const int t = i / DM_COLS, d = i - t * DM_COLS;
      vs[i] = col0 + d < dv ? proj[(size_t)(t0 + t) * ld + v_off + h * dv + col0 + d] : 0.f;
    }
    __syncthreads();
    // Only S passes from one token to the next (one multiply-add a row); the sums and shuffles of
    // neighbouring tokens are independent, so four tokens' worth of them are kept in flight.
#pragma unroll 4
    for (int t = 0; t < nt; ++t) {
      const float* qt = qs + t * dkp;
      const float* kt = ks + t * dkp;
      const float* at = as + t * dkp;
      const float v = vs[t * DM_COLS + threadIdx.x / DM_TPC];
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        if (4 * DM_TPC * i < dk) {
          const float4 k4 = *reinterpret_cast<const float4*>(kt + 4 * DM_TPC * i + 4 * sub);
          const float4 a4 = *reinterpret_cast<const float4*>(at + 4 * DM_TPC * i + 4 * sub);
          S[i * 4 + 0] = fmaf(a4.x, S[i * 4 + 0], k4.x * v);
          S[i * 4 + 1] = fmaf(a4.y, S[i * 4 + 1], k4.y * v);
          S[i * 4 + 2] = fmaf(a4.z, S[i * 4 + 2], k4.z * v);
          S[i * 4 + 3] = fmaf(a4.w, S[i * 4 + 3], k4.w * v);
          if (PHASE == DM_COLLECT) {
            D[i * 4 + 0] *= a4.x; D[i * 4 + 1] *= a4.y; D[i * 4 + 2] *= a4.z; D[i * 4 + 3] *= a4.w;
          } else {
            const float4 q4 = *reinterpret_cast<const float4*>(qt + 4 * DM_TPC * i + 4 * sub);
            acc = fmaf(S[i * 4 + 0], q4.x, acc);
            acc = fmaf(S[i * 4 + 1], q4.y, acc);
            acc = fmaf(S[i * 4 + 2], q4.z, acc);
            acc = fmaf(S[i * 4 + 3], q4.w, acc);
          }
        }
      }
      if (PHASE != DM_COLLECT) {
#pragma unroll
        for (int w = 1; w < DM_TPC; w <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
        if (has_col && sub == 0) out[(size_t)(t0 + t) * H * dv + (size_t)h * dv + c] = acc;
      }
    }
  }
  if (to)
#pragma unroll
    for (int i = 0; i < RPT / 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = 4 * DM_TPC * i + 4 * sub + e;
        if (has_col && r < dk) to[(size_t)r * dv + c] = S[i * 4 + e];
      }
  if (PHASE == DM_COLLECT && blockIdx.z == 0 && threadIdx.x < DM_TPC)
#pragma unroll
    for (int i = 0; i < RPT / 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = 4 * DM_TPC * i + 4 * sub + e;
        if (r < dk) work_decay[((size_t)blockIdx.x * H + h) * dk + r] = D[i * 4 + e];
      }
}

// S_(p+1) = diag(D_p) S_p + L_p over the pieces of one segment; S_p takes L_p's place.  One thread per
// element of S; segments of one piece have nothing to pass on.
__global__ void __launch_bounds__(256)
decay_memory_scan_kernel(const int* __restrict__ cu_pieces, const int4* __restrict__ pieces,
                         const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                         const float* __restrict__ state, float* __restrict__ work,
                         const float* __restrict__ work_decay, int H, int dk, int dv) {
  pdl_begin();
  const int b = blockIdx.x, h = blockIdx.y;
  const int p0 = cu_pieces[b], p1 = cu_pieces[b + 1];
  if (p1 - p0 < 2) return;
  const int n = dk * dv;
  for (int i = blockIdx.z * blockDim.x + threadIdx.x; i < n; i += gridDim.z * blockDim.x) {
    const int r = i / dv;
    float S = seg_start[b] == 0 ? 0.f : state[((size_t)seg_slot[b] * H + h) * n + i];
    for (int p = p0; p < p1; ++p) {
      float* w = work + ((size_t)p * H + h) * n + i;
      if (p + 1 < p1) {
        const float L = *w;
        *w = S;
        S = fmaf(work_decay[((size_t)p * H + h) * dk + r], S, L);
      } else {
        *w = S;
      }
    }
  }
}

// proj: float [M, ld].  mode 0 (gated): gate_bias and gate_low over [H*dk] (float or bfloat16, one flag for
// both).  mode 1 (fixed): decay float [H]; inv_freq float [rot_dim/2] (null or rot_dim 0: no rotation),
// positions int32 [M].  state: float [slots, H, dk, dv].  out: float [M, H*dv].
// n_pieces 0: one block walks a whole segment.  Otherwise pieces int32 [n_pieces, 4], cu_pieces int32 [B+1]
// (first piece of each segment), work float [n_pieces, H, dk, dv], work_decay float [n_pieces, H, dk].
SNK_API int snk_decay_memory(const float* proj, long long ld, int q_off, int k_off, int v_off, int mode,
                             const void* gate_bias, const void* gate_low, int gate_f32, const float* decay,
                             const float* inv_freq, int rot_dim, float k_scale, const int* positions,
                             const int* cu_seqlens, const int* seg_start, const int* seg_slot, float* state,
                             float* out, int B, int H, int dk, int dv, const int* pieces, const int* cu_pieces,
                             int n_pieces, float* work, float* work_decay, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || H > 65535 || dk <= 0 || dk > 256 || dv <= 0 || dv > 32 * 65535) return SNK_ERR_SIZE;
  if (n_pieces < 0 || (n_pieces && (!pieces || !cu_pieces || !work || !work_decay))) return SNK_ERR_SIZE;
  if (n_pieces && ((uintptr_t)pieces & 15)) return SNK_ERR_ALIGN;
  if (mode == DM_GATED) {
    if (!gate_bias || !gate_low) return SNK_ERR_SIZE;
  } else if (mode == DM_FIXED) {
    if (!decay) return SNK_ERR_SIZE;
    if (!inv_freq) rot_dim = 0;
    if (rot_dim < 0 || rot_dim > dk || (rot_dim & 1) || (rot_dim && !positions)) return SNK_ERR_SIZE;
  } else {
    return SNK_ERR_SIZE;
  }
  const int slices = (dv + DM_COLS - 1) / DM_COLS;
  const int dkp = (dk + 4 * DM_TPC - 1) / (4 * DM_TPC) * (4 * DM_TPC);
  const size_t smem = (size_t)(DM_CHUNK * (3 * dkp + DM_COLS)) * sizeof(float);
#define DM_LAUNCH(DKR_, PHASE_, N_)                                                                           \
  do {                                                                                                        \
    auto kernel = decay_memory_kernel<DKR_, PHASE_>;                                                          \
    if (smem > 48 * 1024)                                                                                     \
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                   \
    snk_launch(kernel, dim3(N_, H, slices), dim3(DM_TPC * DM_COLS), smem, stream, proj, ld, q_off, k_off,     \
               v_off, mode, SmallVec{gate_bias, gate_f32}, SmallVec{gate_low, gate_f32}, decay, inv_freq,     \
               rot_dim, k_scale, positions, cu_seqlens, seg_start, seg_slot, state, out, H, dk, dv,           \
               reinterpret_cast<const int4*>(pieces), work, work_decay);                                      \
  } while (0)
#define DM_PHASE(PHASE_, N_)                                                                                  \
  do {                                                                                                        \
    if (dk <= 32) DM_LAUNCH(32, PHASE_, N_);                                                                  \
    else if (dk <= 64) DM_LAUNCH(64, PHASE_, N_);                                                             \
    else if (dk <= 128) DM_LAUNCH(128, PHASE_, N_);                                                           \
    else DM_LAUNCH(256, PHASE_, N_);                                                                          \
  } while (0)
  if (!n_pieces) {
    DM_PHASE(DM_WHOLE, B);
  } else {
    DM_PHASE(DM_COLLECT, n_pieces);
    SNK_LAUNCH_CHECK();
    const int per = (dk * dv + 255) / 256;
    snk_launch(decay_memory_scan_kernel, dim3(B, H, per < 64 ? per : 64), dim3(256), 0, stream, cu_pieces,
               reinterpret_cast<const int4*>(pieces), seg_start, seg_slot, (const float*)state, work,
               (const float*)work_decay, H, dk, dv);
    SNK_LAUNCH_CHECK();
    DM_PHASE(DM_EMIT, n_pieces);
  }
#undef DM_PHASE
#undef DM_LAUNCH
  SNK_LAUNCH_CHECK();
  return 0;
}
