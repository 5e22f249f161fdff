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
// A block serves one (segment, head, 32 column groups of S).  A group is one column, or four where the head
// is wide: the token loop is bound by what it reads from shared memory (q, k and the decays of a thread's
// rows, the same for every column), and four columns a thread share those reads.  Eight neighbouring threads
// share a group: each holds an eighth of its rows in registers over the whole segment, and shuffles add
// their parts of S^T q.  The block meets only to bring the next 32 tokens' q, k and decays into shared memory
// (gates, activations and rotations are evaluated there, off the token loop's chain of dependent
// instructions).
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
#define DM_GROUPS 32           // column groups of S per block (a group: CPT neighbouring columns)
#define DM_TPC 8               // threads per column

enum { DM_GATED = 0, DM_FIXED = 1 };

// q, k and the decay a of row r of head h of one token, from its projections `pr`.
__device__ __forceinline__ void dm_transform(const float* __restrict__ pr, int q_off, int k_off, int h, int r, int dk,
                                             int mode, const SmallVec& gate_bias, const SmallVec& gate_low,
                                             float head_decay, const float* __restrict__ inv_freq, int rot_dim,
                                             float k_scale, int position, float& qv, float& kv, float& av) {
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
      const int half = rot_dim >> 1;
      const int j = r < half ? r : r - half;
      float sn, cs;
      sincosf((float)position * inv_freq[j], &sn, &cs);
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

// The same for every row of the step, once, for the kernels that walk pieces (each of which would otherwise
// evaluate them again for its own 32 columns): prep float [2 or 3][M, H*dk] = q, k and, gated form, a.
__global__ void __launch_bounds__(256)
decay_memory_prepare_kernel(const float* __restrict__ proj, long long ld, int q_off, int k_off, int mode,
                            SmallVec gate_bias, SmallVec gate_low, const float* __restrict__ inv_freq, int rot_dim,
                            float k_scale, const int* __restrict__ positions, float* __restrict__ prep, int M, int H,
                            int dk) {
  pdl_begin();
  const int HD = H * dk;
  const size_t n = (size_t)M * HD;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / HD), j = (int)(i - (size_t)m * HD);
    const int h = j / dk, r = j - h * dk;
    float qv, kv, av;
    dm_transform(proj + (size_t)m * ld, q_off, k_off, h, r, dk, mode, gate_bias, gate_low, 0.f, inv_freq, rot_dim,
                 k_scale, rot_dim ? positions[m] : 0, qv, kv, av);
    prep[i] = qv;
    prep[n + i] = kv;
    if (mode == DM_GATED) prep[2 * n + i] = av;
  }
}

enum { DM_WHOLE = 0, DM_COLLECT = 1, DM_EMIT = 2 };
enum { DM_FIRST = 1, DM_LAST = 2 };

template <int DKR, int PHASE, int CPT>
__global__ void __launch_bounds__(DM_TPC * DM_GROUPS)
decay_memory_kernel(const float* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, int mode,
                    SmallVec gate_bias, SmallVec gate_low, const float* __restrict__ decay,
                    const float* __restrict__ inv_freq, int rot_dim, float k_scale,
                    const int* __restrict__ positions, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                    float* __restrict__ state, float* __restrict__ out, int H, int dk, int dv,
                    const int4* __restrict__ pieces, float* __restrict__ work, float* __restrict__ work_decay,
                    const float* __restrict__ prep, int M) {
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
  constexpr int DM_COLS = DM_GROUPS * CPT;               // columns of S per block
  const int c = blockIdx.z * DM_COLS + threadIdx.x / DM_TPC * CPT;       // my first column
  const bool wide = CPT == 4 && (dv & 3) == 0;           // my four columns as one 16-byte access (all or none exist)
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

  // registers [i*4 + e][j] hold row 4 DM_TPC i + 4 sub + e, column c + j
  float S[RPT][CPT];
#pragma unroll
  for (int i = 0; i < RPT / 4; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = 4 * DM_TPC * i + 4 * sub + e;
      if (CPT == 4 && wide && from && r < dk && c < dv) {
        const float4 s4 = *reinterpret_cast<const float4*>(from + (size_t)r * dv + c);
        S[i * 4 + e][0] = s4.x; S[i * 4 + e][CPT > 1 ? 1 : 0] = s4.y;
        S[i * 4 + e][CPT > 2 ? 2 : 0] = s4.z; S[i * 4 + e][CPT > 3 ? 3 : 0] = s4.w;
      } else {
#pragma unroll
        for (int j = 0; j < CPT; ++j) S[i * 4 + e][j] = (from && r < dk && c + j < dv) ? from[(size_t)r * dv + c + j] : 0.f;
      }
    }
  float D[PHASE == DM_COLLECT ? RPT : 1];                // the product of each row's decays over the piece,
  const bool track = PHASE == DM_COLLECT && blockIdx.z == 0 && threadIdx.x < DM_TPC;   // in one column's threads
  if (PHASE == DM_COLLECT)
#pragma unroll
    for (int i = 0; i < RPT; ++i) D[i] = 1.f;
  const int col0 = blockIdx.z * DM_COLS;
  const float head_decay = mode == DM_FIXED ? decay[h] : 0.f;

  if (PHASE != DM_WHOLE && dkp != dk)                    // rows past dk stay zero (the copies below skip them)
    for (int i = threadIdx.x; i < 3 * DM_CHUNK * dkp; i += blockDim.x) dm_sh[i] = 0.f;
  for (int t0 = row0; t0 < row1; t0 += DM_CHUNK) {
    const int nt = min(DM_CHUNK, row1 - t0);
    __syncthreads();                                     // everyone is done with the previous chunk
    if (PHASE == DM_WHOLE) {
      for (int i = threadIdx.x; i < nt * dkp; i += blockDim.x) {
        const int t = i / dkp, r = i - t * dkp;
        float qv = 0.f, kv = 0.f, av = 0.f;
        if (r < dk)
          dm_transform(proj + (size_t)(t0 + t) * ld, q_off, k_off, h, r, dk, mode, gate_bias, gate_low, head_decay,
                       inv_freq, rot_dim, k_scale, rot_dim ? positions[t0 + t] : 0, qv, kv, av);
        qs[i] = qv;
        ks[i] = kv;
        as[i] = av;
      }
    } else if ((dk & 3) == 0) {                          // prepared rows, four floats at a time
      const int d4 = dk >> 2, p4 = dkp >> 2;
      const size_t n4 = (size_t)M * H * d4;
      const float4* src = reinterpret_cast<const float4*>(prep);
      for (int i = threadIdx.x; i < nt * d4; i += blockDim.x) {
        const int t = i / d4, r4 = i - t * d4;
        const size_t g = ((size_t)(t0 + t) * H + h) * d4 + r4;
        reinterpret_cast<float4*>(qs)[t * p4 + r4] = src[g];
        reinterpret_cast<float4*>(ks)[t * p4 + r4] = src[n4 + g];
        reinterpret_cast<float4*>(as)[t * p4 + r4] =
            mode == DM_GATED ? src[2 * n4 + g] : make_float4(head_decay, head_decay, head_decay, head_decay);
      }
    } else {
      const size_t n = (size_t)M * H * dk;
      for (int i = threadIdx.x; i < nt * dk; i += blockDim.x) {
        const int t = i / dk, r = i - t * dk;
        const size_t g = ((size_t)(t0 + t) * H + h) * dk + r;
        qs[t * dkp + r] = prep[g];
        ks[t * dkp + r] = prep[n + g];
        as[t * dkp + r] = mode == DM_GATED ? prep[2 * n + g] : head_decay;
      }
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
      float v[CPT], acc[CPT];
      if constexpr (CPT == 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(vs + t * DM_COLS + threadIdx.x / DM_TPC * 4);
        v[0] = v4.x; v[1] = v4.y; v[2] = v4.z; v[3] = v4.w;
      } else {
        v[0] = vs[t * DM_COLS + threadIdx.x / DM_TPC];
      }
#pragma unroll
      for (int j = 0; j < CPT; ++j) acc[j] = 0.f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        if (4 * DM_TPC * i < dk) {
          const float4 k4 = *reinterpret_cast<const float4*>(kt + 4 * DM_TPC * i + 4 * sub);
          const float4 a4 = *reinterpret_cast<const float4*>(at + 4 * DM_TPC * i + 4 * sub);
#pragma unroll
          for (int j = 0; j < CPT; ++j) {
            S[i * 4 + 0][j] = fmaf(a4.x, S[i * 4 + 0][j], k4.x * v[j]);
            S[i * 4 + 1][j] = fmaf(a4.y, S[i * 4 + 1][j], k4.y * v[j]);
            S[i * 4 + 2][j] = fmaf(a4.z, S[i * 4 + 2][j], k4.z * v[j]);
            S[i * 4 + 3][j] = fmaf(a4.w, S[i * 4 + 3][j], k4.w * v[j]);
          }
          if (PHASE == DM_COLLECT) {
            if (track) {
            D[i * 4 + 0] *= a4.x; D[i * 4 + 1] *= a4.y; D[i * 4 + 2] *= a4.z; D[i * 4 + 3] *= a4.w;
            }
          } else {
            const float4 q4 = *reinterpret_cast<const float4*>(qt + 4 * DM_TPC * i + 4 * sub);
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
              acc[j] = fmaf(S[i * 4 + 0][j], q4.x, acc[j]);
              acc[j] = fmaf(S[i * 4 + 1][j], q4.y, acc[j]);
              acc[j] = fmaf(S[i * 4 + 2][j], q4.z, acc[j]);
              acc[j] = fmaf(S[i * 4 + 3][j], q4.w, acc[j]);
            }
          }
        }
      }
      if (PHASE != DM_COLLECT) {
        float* orow = out + (size_t)(t0 + t) * H * dv + (size_t)h * dv;
        if constexpr (CPT == 1) {
#pragma unroll
          for (int w = 1; w < DM_TPC; w <<= 1) acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], w);
          if (c < dv && sub == 0) orow[c] = acc[0];
        } else {
          // eight threads hold four partial sums each: two rounds of keep-half-send-half, one plain round;
          // then the threads with an even `sub` hold one column's sum each
          const bool up4 = sub & 4, up2 = sub & 2;
          float keep0 = up4 ? acc[2] : acc[0], keep1 = up4 ? acc[3] : acc[1];
          const float send0 = up4 ? acc[0] : acc[2], send1 = up4 ? acc[1] : acc[3];
          keep0 += __shfl_xor_sync(0xffffffffu, send0, 4);
          keep1 += __shfl_xor_sync(0xffffffffu, send1, 4);
          float sum = up2 ? keep1 : keep0;
          sum += __shfl_xor_sync(0xffffffffu, up2 ? keep0 : keep1, 2);
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          const int mine_col = c + (up4 ? 2 : 0) + (up2 ? 1 : 0);
          if (!(sub & 1) && mine_col < dv) orow[mine_col] = sum;
        }
      }
    }
  }
  if (to)
#pragma unroll
    for (int i = 0; i < RPT / 4; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = 4 * DM_TPC * i + 4 * sub + e;
        if (r >= dk) continue;
        if (CPT == 4 && wide) {
          if (c < dv)
            *reinterpret_cast<float4*>(to + (size_t)r * dv + c) =
                make_float4(S[i * 4 + e][0], S[i * 4 + e][CPT > 1 ? 1 : 0], S[i * 4 + e][CPT > 2 ? 2 : 0],
                            S[i * 4 + e][CPT > 3 ? 3 : 0]);
        } else {
#pragma unroll
          for (int j = 0; j < CPT; ++j)
            if (c + j < dv) to[(size_t)r * dv + c + j] = S[i * 4 + e][j];
        }
      }
  if (track)
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
    float* w = work + ((size_t)p0 * H + h) * n + i;
    const float* d = work_decay + ((size_t)p0 * H + h) * dk + r;
    const size_t wstep = (size_t)H * n, dstep = (size_t)H * dk;
    const int last = p1 - 1 - p0;
    for (int p = 0; p < last; p += 8) {                  // eight pieces' loads in flight, then their chain
      float L[8], D[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (p + j < last) {
          L[j] = w[(p + j) * wstep];
          D[j] = d[(p + j) * dstep];
        }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (p + j < last) {
          w[(p + j) * wstep] = S;
          S = fmaf(D[j], S, L[j]);
        }
    }
    w[last * wstep] = S;
  }
}

// proj: float [M, ld].  mode 0 (gated): gate_bias and gate_low over [H*dk] (float or bfloat16, one flag for
// both).  mode 1 (fixed): decay float [H]; inv_freq float [rot_dim/2] (null or rot_dim 0: no rotation),
// positions int32 [M].  state: float [slots, H, dk, dv].  out: float [M, H*dv].
// n_pieces 0: one block walks a whole segment.  Otherwise pieces int32 [n_pieces, 4], cu_pieces int32 [B+1]
// (first piece of each segment), work float [n_pieces, H, dk, dv], work_decay float [n_pieces, H, dk], prep
// float [3, M, H*dk] (fixed form: 2), M the rows of proj.
SNK_API int snk_decay_memory(const float* proj, long long ld, int q_off, int k_off, int v_off, int mode,
                             const void* gate_bias, const void* gate_low, int gate_f32, const float* decay,
                             const float* inv_freq, int rot_dim, float k_scale, const int* positions,
                             const int* cu_seqlens, const int* seg_start, const int* seg_slot, float* state,
                             float* out, int B, int H, int dk, int dv, const int* pieces, const int* cu_pieces,
                             int n_pieces, float* work, float* work_decay, float* prep, int M,
                             cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || H > 65535 || dk <= 0 || dk > 256 || dv <= 0 || dv > 32 * 65535) return SNK_ERR_SIZE;
  if (n_pieces < 0 || (n_pieces && (!pieces || !cu_pieces || !work || !work_decay || !prep || M <= 0))) return SNK_ERR_SIZE;
  if (n_pieces && (((uintptr_t)pieces | (uintptr_t)prep) & 15)) return SNK_ERR_ALIGN;
  if (mode == DM_GATED) {
    if (!gate_bias || !gate_low) return SNK_ERR_SIZE;
  } else if (mode == DM_FIXED) {
    if (!decay) return SNK_ERR_SIZE;
    if (!inv_freq) rot_dim = 0;
    if (rot_dim < 0 || rot_dim > dk || (rot_dim & 1) || (rot_dim && !positions)) return SNK_ERR_SIZE;
  } else {
    return SNK_ERR_SIZE;
  }
  // four columns a thread where the head is wide enough to fill a block that way, else one
  const int cpt = dv > 2 * DM_GROUPS ? 4 : 1;
  const int cols = DM_GROUPS * cpt;
  const int slices = (dv + cols - 1) / cols;
  const int dkp = (dk + 4 * DM_TPC - 1) / (4 * DM_TPC) * (4 * DM_TPC);
  const size_t smem = (size_t)(DM_CHUNK * (3 * dkp + cols)) * sizeof(float);
#define DM_LAUNCH_C(DKR_, PHASE_, N_, CPT_)                                                                   \
  do {                                                                                                        \
    auto kernel = decay_memory_kernel<DKR_, PHASE_, CPT_>;                                                    \
    if (smem > 48 * 1024)                                                                                     \
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                   \
    snk_launch(kernel, dim3(N_, H, slices), dim3(DM_TPC * DM_GROUPS), smem, stream, proj, ld, q_off, k_off,   \
               v_off, mode, SmallVec{gate_bias, gate_f32}, SmallVec{gate_low, gate_f32}, decay, inv_freq,     \
               rot_dim, k_scale, positions, cu_seqlens, seg_start, seg_slot, state, out, H, dk, dv,           \
               reinterpret_cast<const int4*>(pieces), work, work_decay, (const float*)prep, M);               \
  } while (0)
#define DM_LAUNCH(DKR_, PHASE_, N_)                                                                           \
  do {                                                                                                        \
    if (cpt == 4) DM_LAUNCH_C(DKR_, PHASE_, N_, 4);                                                           \
    else DM_LAUNCH_C(DKR_, PHASE_, N_, 1);                                                                    \
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
    const size_t cells = (size_t)M * H * dk;
    const size_t blocks = (cells + 255) / 256;
    snk_launch(decay_memory_prepare_kernel, dim3((unsigned)(blocks < 148 * 16 ? blocks : 148 * 16)), dim3(256), 0, stream,
               proj, ld, q_off, k_off, mode, SmallVec{gate_bias, gate_f32}, SmallVec{gate_low, gate_f32}, inv_freq,
               rot_dim, k_scale, positions, prep, M, H, dk);
    SNK_LAUNCH_CHECK();
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
#undef DM_LAUNCH_C
  SNK_LAUNCH_CHECK();
  return 0;
}
