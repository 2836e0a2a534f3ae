// Retention: linear attention with a fixed decay per head and neither softmax nor denominator, in 32-bit arithmetic
// whatever the storage type.
//
// Per request and head the state is a matrix S [D x V], zero at the start.  For every token, in order,
//   q, k: the head's query and key, their first `rot_dims` entries rotated in pairs (entry i with entry
//         i + rot_dims/2) by the angle position * freqs[i]; k then times k_scale
//   S <- decay_h S + k v^T;   y = S^T q
// The decay comes as 1 - decay_h (made on the host in 64-bit and rounded once): S - (1 - decay) S keeps the digits of
// a decay near 1 that the rounded decay itself has lost.  A segment's rows are walked in order from the request's
// state, so a position's values are the same bits whether its prompt came whole, in portions or token by token.
//
// grid (column blocks, heads, segments).  A block owns CB columns of S; a thread holds CPT of them (4, 2 where a
// column is long, 1 in steps of short segments), each spread over L lanes: lane l holds the rows d = l, l + L, ... of
// its columns in registers, so one key or query entry read from shared memory serves CPT columns.  Rows come through
// shared memory TC at a time (16; 4 in steps of short segments): k and q as 32-bit (rotated there, one sine and
// cosine per pair serving both), a lane's entries side by side (16-byte loads, the lanes' runs padded apart so that
// they meet no bank twice), and the block's slice of v; the next TC rows are on their way from memory, into
// registers, while these are walked.  A column's L partial sums are added in a tree of shuffles whose first steps
// halve the columns a lane still carries, so CPT columns take log2(L) + CPT - 2 shuffles and every form adds in the
// same order.  State of a slot: S as [H][V][D].
//
// One long prompt offers heads x columns of parallel work only, and its rows wait on one another.  Where a step's
// states are few and its longest segment is long, segments are cut into pieces of `piece_rows` rows that run side by
// side (grid.z = segments x pieces), in three launches: every piece but a segment's last walks its rows from a zero
// state and leaves the end state (no y); the start states follow one after the other,
// start[p + 1] = decay^piece_rows start[p] + end[p], start[0] the request's state; then every piece walks its rows
// again from its start state and writes y, the last piece the request's state.  Twice the arithmetic for many times
// the parallel work; against the walk in one piece the results differ by rounding only.
#include "common.cuh"

namespace cbis {

constexpr int kRetRows = 16;      // rows of a batch for long segments
constexpr int kRetRowsShort = 4;  // rows of a batch where no segment of the step is longer (decode steps)

__host__ __device__ inline int ret_lanes(int D) { return D <= 256 ? 8 : 16; }
// floats between the runs of two lanes in a staged row: a multiple of 4 whose quarter is odd
__host__ __device__ constexpr int ret_run(int npl) { return ((npl + 3) / 4) % 2 ? (npl + 3) / 4 * 4 : (npl + 3) / 4 * 4 + 4; }

enum { kRetWhole = 0, kRetEnds = 1, kRetFromStarts = 2 };

template <typename TT, int NPL, int L, int CPT, int CB, int TC, int MODE>
__global__ void __launch_bounds__(CB / CPT * L)
retention_kernel(const TT* qkv, int ld, int q_off, int k_off, int v_off, const int* positions,
                 const float* __restrict__ freqs, int rot_dims, float k_scale, const float* __restrict__ one_minus_decay,
                 float* state, long long slot_stride, const int* seg_slot, const int* cu_rows, float* y, int y_ld, int H,
                 int D, int V, int n_pieces, int piece_rows, float* starts) {
  static_assert(CPT == 1 || CPT == 2 || CPT == 4, "columns a thread");
  // a thread of one column reads its entries one by one, a stride of L apart: the rows are staged as they are
  constexpr bool kRuns = CPT > 1;
  constexpr int DP = NPL * L, RUN = kRuns ? ret_run(NPL) : NPL, DPP = RUN * L, THREADS = CB / CPT * L;
  constexpr int KQ_PER = (TC * DP + THREADS - 1) / THREADS, V_PER = (TC * CB + THREADS - 1) / THREADS;
  extern __shared__ __align__(16) float smem[];
  float* ks = smem;                      // [TC][L][RUN]: entry d at (d % L) * RUN + d / L (one column a thread: at d)
  float* qs = ks + TC * DPP;             // the same
  float* vs = qs + TC * DPP;             // [TC][CB]
  float* nums = vs + TC * CB;            // [TC][CB]
  float* pos = nums + TC * CB;           // [TC]
  pdl_trigger();
  const int xb = blockIdx.x, h = blockIdx.y;
  int s = blockIdx.z, piece = 0;
  if (MODE != kRetWhole) {
    piece = s % n_pieces;
    s /= n_pieces;
  }
  const float om = one_minus_decay[h];
  pdl_wait();
  int row0 = cu_rows[s], n_rows = cu_rows[s + 1] - row0;
  bool last = true;                  // the piece that holds the segment's last row leaves the request's state
  if (MODE != kRetWhole) {
    const int before = piece * piece_rows;
    last = before + piece_rows >= n_rows;
    if (before >= n_rows || (MODE == kRetEnds && last)) return;
    row0 += before;
    n_rows = min(piece_rows, n_rows - before);
  }
  if (n_rows <= 0) return;
  const int tid = threadIdx.x;
  const int l = tid % L, g = tid / L;
  const int col = xb * CB + g * CPT;           // the first of this thread's columns
  const size_t at = ((size_t)h * V + (col < V ? col : 0)) * D;       // its place in a state
  float* sp = state + (long long)seg_slot[s] * slot_stride + at;
  const size_t per_state = (size_t)H * V * D;
  const float* from = MODE == kRetFromStarts ? starts + ((size_t)s * n_pieces + piece) * per_state + at : sp;
  float* into = MODE == kRetEnds ? starts + ((size_t)s * n_pieces + piece + 1) * per_state + at : sp;
  float S[CPT][NPL];
#pragma unroll
  for (int j = 0; j < CPT; ++j) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = l + L * i;
      S[j][i] = (MODE != kRetEnds && col + j < V && d < D) ? from[(size_t)j * D + d] : 0.f;
    }
  }
  const TT* qrow = qkv + (size_t)row0 * ld + q_off + h * D;
  const TT* krow = qkv + (size_t)row0 * ld + k_off + h * D;
  const TT* vrow = qkv + (size_t)row0 * ld + v_off + h * V + xb * CB;
  const int vcols = min(CB, V - xb * CB);
  const int half = rot_dims / 2;
  auto staged = [](int d) { return kRuns ? (d % L) * RUN + d / L : d; };

  // what this thread fetches of a batch of rows: entries of k and q (row t = idx / DP, entry d = idx % DP), of the
  // block's slice of v, and (the first TC threads) a row's position
  float r_k[KQ_PER], r_q[KQ_PER], r_v[V_PER], r_pos = 0.f;
  auto fetch = [&](int first) {
    const int tc = min(TC, n_rows - first);
#pragma unroll
    for (int j = 0; j < KQ_PER; ++j) {
      const int idx = tid + THREADS * j, t = idx / DP, d = idx % DP;
      const bool ok = t < tc && d < D;
      r_k[j] = ok ? to_f32(krow[(size_t)(first + t) * ld + d]) : 0.f;
      r_q[j] = (MODE != kRetEnds && ok) ? to_f32(qrow[(size_t)(first + t) * ld + d]) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < V_PER; ++j) {
      const int idx = tid + THREADS * j, t = idx / CB, cc = idx % CB;
      r_v[j] = (t < tc && cc < vcols) ? to_f32(vrow[(size_t)(first + t) * ld + cc]) : 0.f;
    }
    if (tid < tc) r_pos = (float)positions[row0 + first + tid];
  };
  fetch(0);
  for (int first = 0; first < n_rows; first += TC) {
    const int tc = min(TC, n_rows - first);
    __syncthreads();                 // the rows staged before have been used
#pragma unroll
    for (int j = 0; j < KQ_PER; ++j) {
      const int idx = tid + THREADS * j;
      if (idx < TC * DP) {
        const int at_s = (idx / DP) * DPP + staged(idx % DP);
        ks[at_s] = r_k[j] * k_scale;      // a rotation is linear: the key's scale may come first
        if (MODE != kRetEnds) qs[at_s] = r_q[j];
      }
    }
#pragma unroll
    for (int j = 0; j < V_PER; ++j) {
      const int idx = tid + THREADS * j;
      if (idx < TC * CB) vs[idx] = r_v[j];
    }
    if (tid < TC) pos[tid] = r_pos;
    __syncthreads();
    if (first + TC < n_rows) fetch(first + TC);      // in flight while these rows are turned and walked
    // the rotation: one angle per (row, pair) serves the key and the query
    for (int u = tid; u < tc * half; u += THREADS) {
      const int t = u / half, i = u % half;
      float sn, cs;
      sincosf(pos[t] * freqs[i], &sn, &cs);
      float* kt = ks + t * DPP;
      float* qt = qs + t * DPP;
      const int ia = staged(i), ib = staged(i + half);
      const float ka = kt[ia], kb = kt[ib];
      kt[ia] = ka * cs - kb * sn;
      kt[ib] = kb * cs + ka * sn;
      if (MODE != kRetEnds) {
        const float qa = qt[ia], qb = qt[ib];
        qt[ia] = qa * cs - qb * sn;
        qt[ib] = qb * cs + qa * sn;
      }
    }
    __syncthreads();
#pragma unroll 2
    for (int t = 0; t < tc; ++t) {
      float kk[(NPL + 3) / 4 * 4], qq[(NPL + 3) / 4 * 4], vv[CPT];
      if constexpr (kRuns) {
        const float4* k4 = reinterpret_cast<const float4*>(ks + t * DPP + l * RUN);
        const float4* q4 = reinterpret_cast<const float4*>(qs + t * DPP + l * RUN);
#pragma unroll
        for (int i = 0; i < (NPL + 3) / 4; ++i) {
          const float4 a = k4[i];
          kk[4 * i] = a.x, kk[4 * i + 1] = a.y, kk[4 * i + 2] = a.z, kk[4 * i + 3] = a.w;
          if (MODE != kRetEnds) {
            const float4 b = q4[i];
            qq[4 * i] = b.x, qq[4 * i + 1] = b.y, qq[4 * i + 2] = b.z, qq[4 * i + 3] = b.w;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          kk[i] = ks[t * DPP + l + L * i];
          if (MODE != kRetEnds) qq[i] = qs[t * DPP + l + L * i];
        }
      }
      if constexpr (CPT == 4) {
        const float4 a = *reinterpret_cast<const float4*>(vs + t * CB + g * 4);
        vv[0] = a.x, vv[1] = a.y, vv[2] = a.z, vv[3] = a.w;
      } else if constexpr (CPT == 2) {
        const float2 a = *reinterpret_cast<const float2*>(vs + t * CB + g * 2);
        vv[0] = a.x, vv[1] = a.y;
      } else {
        vv[0] = vs[t * CB + g];
      }
      if constexpr (MODE == kRetEnds) {          // the end state only: no y
#pragma unroll
        for (int i = 0; i < NPL; ++i)
#pragma unroll
          for (int j = 0; j < CPT; ++j) S[j][i] = fmaf(vv[j], kk[i], fmaf(-om, S[j][i], S[j][i]));
      } else {
        float a0[CPT], a1[CPT], acc[CPT];
#pragma unroll
        for (int j = 0; j < CPT; ++j) a0[j] = a1[j] = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
#pragma unroll
          for (int j = 0; j < CPT; ++j) {
            S[j][i] = fmaf(vv[j], kk[i], fmaf(-om, S[j][i], S[j][i]));
            if (i & 1) a1[j] = fmaf(S[j][i], qq[i], a1[j]);
            else a0[j] = fmaf(S[j][i], qq[i], a0[j]);
          }
        }
#pragma unroll
        for (int j = 0; j < CPT; ++j) acc[j] = a0[j] + a1[j];
        // the sum over a column's lanes; a lane passes on the columns its partner keeps
        float sum;
        int mine = 0, o = 1;                       // the column (of CPT) whose sum this lane ends with
        if constexpr (CPT == 4) {
          const bool hi = l & 1, hi2 = l & 2;
          float k0 = hi ? acc[2] : acc[0], k1 = hi ? acc[3] : acc[1];
          k0 += __shfl_xor_sync(0xffffffffu, hi ? acc[0] : acc[2], 1);
          k1 += __shfl_xor_sync(0xffffffffu, hi ? acc[1] : acc[3], 1);
          sum = (hi2 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, hi2 ? k0 : k1, 2);
          mine = 2 * (l & 1) + ((l >> 1) & 1);
          o = 4;
        } else if constexpr (CPT == 2) {
          const bool hi = l & 1;
          sum = (hi ? acc[1] : acc[0]) + __shfl_xor_sync(0xffffffffu, hi ? acc[0] : acc[1], 1);
          mine = l & 1;
          o = 2;
        } else {
          sum = acc[0];
        }
#pragma unroll
        for (; o < L; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (l < CPT) nums[t * CB + g * CPT + mine] = sum;
      }
    }
    if constexpr (MODE != kRetEnds) {
      __syncthreads();
      for (int i = tid; i < tc * CB; i += THREADS) {
        const int t = i / CB, cc = i % CB;
        if (cc < vcols) y[(size_t)(row0 + first + t) * y_ld + h * V + xb * CB + cc] = nums[i];
      }
    }
  }
  if (MODE != kRetFromStarts || last) {
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int d = l + L * i;
        if (col + j < V && d < D) into[(size_t)j * D + d] = S[j][i];
      }
    }
  }
}

// The start states of a cut segment's pieces, one after the other: starts[s][0] is the request's state, starts[s][p]
// (which holds the end state, from zero, of piece p - 1) becomes decay^piece_rows starts[s][p - 1] + itself.
// grid (blocks of elements, segments); a thread owns one element of the state.
__global__ void __launch_bounds__(256)
retention_starts_kernel(float* starts, const float* state, long long slot_stride, const int* seg_slot, const int* cu_rows,
                        const float* __restrict__ decay_piece, int n_pieces, int piece_rows, int VD, int HVD) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x;
  const int n_rows = cu_rows[s + 1] - cu_rows[s];
  if (e >= HVD || n_rows <= 0) return;
  const int np = (n_rows + piece_rows - 1) / piece_rows;
  const float dp = decay_piece[e / VD];
  float* st = starts + (size_t)s * n_pieces * HVD + e;
  float cur = state[(long long)seg_slot[s] * slot_stride + e];
  st[0] = cur;
  int p = 1;
  for (; p + 4 <= np; p += 4) {       // four ends on their way at a time
    const float e0 = st[(size_t)p * HVD], e1 = st[(size_t)(p + 1) * HVD], e2 = st[(size_t)(p + 2) * HVD],
                e3 = st[(size_t)(p + 3) * HVD];
    st[(size_t)p * HVD] = cur = fmaf(dp, cur, e0);
    st[(size_t)(p + 1) * HVD] = cur = fmaf(dp, cur, e1);
    st[(size_t)(p + 2) * HVD] = cur = fmaf(dp, cur, e2);
    st[(size_t)(p + 3) * HVD] = cur = fmaf(dp, cur, e3);
  }
  for (; p < np; ++p) st[(size_t)p * HVD] = cur = fmaf(dp, cur, st[(size_t)p * HVD]);
}

template <typename TT>
static int launch_retention(const void* qkv, int ld, int q_off, int k_off, int v_off, const int* positions,
                            const float* freqs, int rot_dims, float k_scale, const float* one_minus_decay, float* state,
                            long long slot_stride, const int* seg_slot, const int* cu_rows, float* y, int y_ld, int S,
                            int H, int D, int V, int max_seg_rows, int n_pieces, int piece_rows, float* starts,
                            const float* decay_piece, cudaStream_t st) {
  const int L = ret_lanes(D);
  const int npl = (D + L - 1) / L;
  // long segments: 16 threads a lane of 4 columns each (2 where a column takes more than 16 registers a lane),
  // walking 16 rows a batch; steps of short segments (decoding): blocks of 32 columns, one a thread, and batches of 4
  const bool shorts = max_seg_rows > 0 && max_seg_rows <= kRetRowsShort;
#define CBIS_RET_AS(NPL, LL, CPT, TCC, MODE, Z)                                                                      \
  do {                                                                                                               \
    constexpr int CBB = CPT == 1 ? 32 : 16 * CPT;                                                                    \
    const size_t smem = ((size_t)2 * TCC * (CPT > 1 ? ret_run(NPL) : NPL) * LL + 2 * TCC * CBB + TCC) * sizeof(float); \
    if (smem > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(retention_kernel<TT, NPL, LL, CPT, CBB, TCC, MODE>,                                       \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                  \
    err = launch_pdl(retention_kernel<TT, NPL, LL, CPT, CBB, TCC, MODE>, dim3((V + CBB - 1) / CBB, H, Z),            \
                     dim3(CBB / CPT * LL), smem, st, (const TT*)qkv, ld, q_off, k_off, v_off, positions, freqs,      \
                     rot_dims, k_scale, one_minus_decay, state, slot_stride, seg_slot, cu_rows, y, y_ld, H, D, V,    \
                     n_pieces, piece_rows, starts);                                                                  \
  } while (0)
#define CBIS_RET(NPL, LL)                                                                                            \
  do {                                                                                                               \
    cudaError_t err = cudaSuccess;                                                                                   \
    constexpr int CPT = NPL <= 16 ? 4 : 2;                                                                           \
    if (n_pieces > 1) {                                                                                              \
      const int HVD = H * V * D;                                                                                     \
      CBIS_RET_AS(NPL, LL, CPT, kRetRows, kRetEnds, S * n_pieces);                                                   \
      if (err != cudaSuccess) return (int)err;                                                                       \
      err = launch_pdl(retention_starts_kernel, dim3((HVD + 255) / 256, S), dim3(256), 0, st, starts,                \
                       (const float*)state, slot_stride, seg_slot, cu_rows, decay_piece, n_pieces, piece_rows,       \
                       V * D, HVD);                                                                                  \
      if (err != cudaSuccess) return (int)err;                                                                       \
      CBIS_RET_AS(NPL, LL, CPT, kRetRows, kRetFromStarts, S * n_pieces);                                             \
      return (int)err;                                                                                               \
    }                                                                                                                \
    if (shorts) {                                                                                                    \
      CBIS_RET_AS(NPL, LL, 1, kRetRowsShort, kRetWhole, S);                                                          \
      return (int)err;                                                                                               \
    }                                                                                                                \
    CBIS_RET_AS(NPL, LL, CPT, kRetRows, kRetWhole, S);                                                               \
    return (int)err;                                                                                                 \
  } while (0)
  if (L == 8) {
    if (npl <= 2) CBIS_RET(2, 8);
    if (npl <= 4) CBIS_RET(4, 8);
    if (npl <= 6) CBIS_RET(6, 8);
    if (npl <= 8) CBIS_RET(8, 8);
    if (npl <= 12) CBIS_RET(12, 8);
    if (npl <= 16) CBIS_RET(16, 8);
    if (npl <= 24) CBIS_RET(24, 8);
    CBIS_RET(32, 8);
  }
  if (npl <= 24) CBIS_RET(24, 16);
  CBIS_RET(32, 16);
#undef CBIS_RET
#undef CBIS_RET_AS
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_retention_max_dim() { return 512; }

// qkv [T, ld] of the compute type: q at columns q_off + h * D, k at k_off + h * D, v at v_off + h * V; positions
// [T]; freqs [rot_dims / 2] 32-bit; one_minus_decay [H] 32-bit; max_seg_rows: the longest segment of the step (0:
// unknown); y [T, y_ld] 32-bit, H * V columns; state: 32-bit, H * V * D per slot at `state + slot * slot_stride`.
// n_pieces > 1: segments are cut into up to n_pieces pieces of piece_rows rows (a multiple of 32, and
// n_pieces * piece_rows >= max_seg_rows); starts: 32-bit scratch [n_segments * n_pieces][H * V * D]; decay_piece
// [H]: decay^piece_rows.
CBIS_EXPORT int cbis_retention(const void* qkv, int ld, int q_off, int k_off, int v_off, const int* positions,
                               const float* freqs, int rot_dims, float k_scale, const float* one_minus_decay,
                               float* state, long long slot_stride, const int* seg_slot, const int* cu_rows, float* y,
                               int y_ld, int n_segments, int H, int D, int V, int dtype, void* stream, int max_seg_rows,
                               int n_pieces, int piece_rows, float* starts, const float* decay_piece) {
  if (n_segments <= 0) return CBIS_OK;
  if (H <= 0 || D <= 0 || V <= 0 || D > 512) return CBIS_ERR_BAD_SIZE;
  if (rot_dims < 0 || rot_dims > D || rot_dims % 2 || (rot_dims > 0 && !freqs)) return CBIS_ERR_BAD_SIZE;
  if (n_segments > 65535 || H > 65535) return CBIS_ERR_TOO_LARGE;
  if (n_pieces > 1) {
    if (piece_rows <= 0 || piece_rows % kRetRows || !starts || !decay_piece || max_seg_rows <= 0 ||
        (long long)n_pieces * piece_rows < max_seg_rows)
      return CBIS_ERR_BAD_SIZE;
    if ((long long)n_segments * n_pieces > 65535) return CBIS_ERR_TOO_LARGE;
  } else {
    n_pieces = 1;
  }
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == CBIS_F32)
    return launch_retention<float>(qkv, ld, q_off, k_off, v_off, positions, freqs, rot_dims, k_scale, one_minus_decay,
                                   state, slot_stride, seg_slot, cu_rows, y, y_ld, n_segments, H, D, V, max_seg_rows, n_pieces,
                                   piece_rows, starts, decay_piece, st);
  if (dtype == CBIS_BF16)
    return launch_retention<__nv_bfloat16>(qkv, ld, q_off, k_off, v_off, positions, freqs, rot_dims, k_scale,
                                           one_minus_decay, state, slot_stride, seg_slot, cu_rows, y, y_ld, n_segments,
                                           H, D, V, max_seg_rows, n_pieces, piece_rows, starts, decay_piece, st);
  return CBIS_ERR_BAD_DTYPE;
}
