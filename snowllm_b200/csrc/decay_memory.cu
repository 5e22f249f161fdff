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
#include "common.cuh"

#define DM_CHUNK 32            // tokens brought in at a time
#define DM_COLS 32             // columns of S per block
#define DM_TPC 8               // threads per column

enum { DM_GATED = 0, DM_FIXED = 1 };

template <int DKR>
__global__ void __launch_bounds__(DM_TPC * DM_COLS)
decay_memory_kernel(const float* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, int mode,
                    SmallVec gate_bias, SmallVec gate_low, const float* __restrict__ decay,
                    const float* __restrict__ inv_freq, int rot_dim, float k_scale,
                    const int* __restrict__ positions, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ seg_start, const int* __restrict__ seg_slot,
                    float* __restrict__ state, float* __restrict__ out, int H, int dk, int dv) {
  pdl_begin();
  extern __shared__ __align__(16) float dm_sh[];
  constexpr int RPT = DKR / DM_TPC;                      // rows of S per thread
  const int b = blockIdx.x, h = blockIdx.y;
  const int sub = threadIdx.x & (DM_TPC - 1);            // which share of the column's rows
  const int c = blockIdx.z * DM_COLS + threadIdx.x / DM_TPC;
  const bool has_col = c < dv;
  const int dkp = (dk + 4 * DM_TPC - 1) / (4 * DM_TPC) * (4 * DM_TPC);
  float* qs = dm_sh;                                     // [DM_CHUNK][dkp]
  float* ks = qs + DM_CHUNK * dkp;                       // [DM_CHUNK][dkp]
  float* as = ks + DM_CHUNK * dkp;                       // [DM_CHUNK][dkp]  decay of each row of S
  float* vs = as + DM_CHUNK * dkp;                       // [DM_CHUNK][DM_COLS]

  const int row0 = cu_seqlens[b], row1 = cu_seqlens[b + 1];
  const bool fresh = seg_start[b] == 0;
  float* Ss = state + ((size_t)seg_slot[b] * H + h) * dk * dv;

  // register i*4 + e holds row 4 DM_TPC i + 4 sub + e
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT / 4; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = 4 * DM_TPC * i + 4 * sub + e;
      S[i * 4 + e] = (!fresh && has_col && r < dk) ? Ss[(size_t)r * dv + c] : 0.f;
    }
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
          const float4 q4 = *reinterpret_cast<const float4*>(qt + 4 * DM_TPC * i + 4 * sub);
          const float4 a4 = *reinterpret_cast<const float4*>(at + 4 * DM_TPC * i + 4 * sub);
          S[i * 4 + 0] = fmaf(a4.x, S[i * 4 + 0], k4.x * v); acc = fmaf(S[i * 4 + 0], q4.x, acc);
          S[i * 4 + 1] = fmaf(a4.y, S[i * 4 + 1], k4.y * v); acc = fmaf(S[i * 4 + 1], q4.y, acc);
          S[i * 4 + 2] = fmaf(a4.z, S[i * 4 + 2], k4.z * v); acc = fmaf(S[i * 4 + 2], q4.z, acc);
          S[i * 4 + 3] = fmaf(a4.w, S[i * 4 + 3], k4.w * v); acc = fmaf(S[i * 4 + 3], q4.w, acc);
        }
      }
#pragma unroll
      for (int w = 1; w < DM_TPC; w <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, w);
      if (has_col && sub == 0) out[(size_t)(t0 + t) * H * dv + (size_t)h * dv + c] = acc;
    }
  }
#pragma unroll
  for (int i = 0; i < RPT / 4; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = 4 * DM_TPC * i + 4 * sub + e;
      if (has_col && r < dk) Ss[(size_t)r * dv + c] = S[i * 4 + e];
    }
}

// proj: float [M, ld].  mode 0 (gated): gate_bias and gate_low over [H*dk] (float or bfloat16, one flag for
// both).  mode 1 (fixed): decay float [H]; inv_freq float [rot_dim/2] (null or rot_dim 0: no rotation),
// positions int32 [M].  state: float [slots, H, dk, dv].  out: float [M, H*dv].
SNK_API int snk_decay_memory(const float* proj, long long ld, int q_off, int k_off, int v_off, int mode,
                             const void* gate_bias, const void* gate_low, int gate_f32, const float* decay,
                             const float* inv_freq, int rot_dim, float k_scale, const int* positions,
                             const int* cu_seqlens, const int* seg_start, const int* seg_slot, float* state,
                             float* out, int B, int H, int dk, int dv, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || H > 65535 || dk <= 0 || dk > 256 || dv <= 0 || dv > 32 * 65535) return SNK_ERR_SIZE;
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
  dim3 grid(B, H, slices);
#define DM_LAUNCH(DKR_)                                                                                       \
  do {                                                                                                        \
    if (smem > 48 * 1024)                                                                                     \
      cudaFuncSetAttribute(decay_memory_kernel<DKR_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    snk_launch(decay_memory_kernel<DKR_>, dim3(grid), dim3(DM_TPC * DM_COLS), smem, stream, proj, ld, q_off,   \
               k_off, v_off, mode, SmallVec{gate_bias, gate_f32}, SmallVec{gate_low, gate_f32}, decay,        \
               inv_freq, rot_dim, k_scale, positions, cu_seqlens, seg_start, seg_slot, state, out, H, dk, dv); \
  } while (0)
  if (dk <= 32) DM_LAUNCH(32);
  else if (dk <= 64) DM_LAUNCH(64);
  else if (dk <= 128) DM_LAUNCH(128);
  else DM_LAUNCH(256);
#undef DM_LAUNCH
  SNK_LAUNCH_CHECK();
  return 0;
}
