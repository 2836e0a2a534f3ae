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
// grid (column blocks, heads, segments).  A block owns CB columns of S (16, or 32 in steps of short segments); a
// column is spread over L lanes, lane l holding the rows d = l, l + L, ... in registers.  Rows come through shared
// memory TC at a time (32; 4 in steps of short segments): k and q as 32-bit (rotated there, one sine and cosine
// per pair serving both), and the block's slice of v; the next TC rows are on their way from memory, into registers,
// while these are walked.  State of a slot: S as [H][V][D].
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

constexpr int kRetRows = 32;      // rows of a batch for long segments
constexpr int kRetRowsShort = 4;  // rows of a batch where no segment of the step is longer (decode steps)

__host__ __device__ inline int ret_lanes(int D) { return D <= 256 ? 8 : 16; }

enum { kRetWhole = 0, kRetEnds = 1, kRetFromStarts = 2 };

template <typename TT, int NPL, int L, int CB, int TC, int MODE>
__global__ void __launch_bounds__(CB * L)
retention_kernel(const TT* qkv, int ld, int q_off, int k_off, int v_off, const int* positions,
                 const float* __restrict__ freqs, int rot_dims, float k_scale, const float* __restrict__ one_minus_decay,
                 float* state, long long slot_stride, const int* seg_slot, const int* cu_rows, float* y, int y_ld, int H,
                 int D, int V, int n_pieces, int piece_rows, float* starts) {
  constexpr int DP = NPL * L, THREADS = CB * L;
  constexpr int KQ_PER = (TC * DP + THREADS - 1) / THREADS, V_PER = (TC * CB + THREADS - 1) / THREADS;
  extern __shared__ float smem[];
  float* ks = smem;                      // [TC][DP]
  float* qs = ks + TC * DP;              // [TC][DP]
  float* vs = qs + TC * DP;              // [TC][CB]
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
  const int l = tid % L, c = tid / L;
  const int col = xb * CB + c;
  const bool live = col < V;
  const size_t at = ((size_t)h * V + (live ? col : 0)) * D;       // the column's place in a state
  float* sp = state + (long long)seg_slot[s] * slot_stride + at;
  const size_t per_state = (size_t)H * V * D;
  const float* from = MODE == kRetFromStarts ? starts + ((size_t)s * n_pieces + piece) * per_state + at : sp;
  float* into = MODE == kRetEnds ? starts + ((size_t)s * n_pieces + piece + 1) * per_state + at : sp;
  float S[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int d = l + L * i;
    S[i] = (MODE != kRetEnds && live && d < D) ? from[d] : 0.f;
  }
  const TT* qrow = qkv + (size_t)row0 * ld + q_off + h * D;
  const TT* krow = qkv + (size_t)row0 * ld + k_off + h * D;
  const TT* vrow = qkv + (size_t)row0 * ld + v_off + h * V + xb * CB;
  const int vcols = min(CB, V - xb * CB);
  const int half = rot_dims / 2;

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
        ks[idx] = r_k[j] * k_scale;      // a rotation is linear: the key's scale may come first
        if (MODE != kRetEnds) qs[idx] = r_q[j];
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
      float* kt = ks + t * DP;
      float* qt = qs + t * DP;
      const float ka = kt[i], kb = kt[i + half];
      kt[i] = ka * cs - kb * sn;
      kt[i + half] = kb * cs + ka * sn;
      if (MODE != kRetEnds) {
        const float qa = qt[i], qb = qt[i + half];
        qt[i] = qa * cs - qb * sn;
        qt[i + half] = qb * cs + qa * sn;
      }
    }
    __syncthreads();
    if constexpr (MODE == kRetEnds) {          // the end state only: no y
#pragma unroll 4
      for (int t = 0; t < tc; ++t) {
        const float vv = vs[t * CB + c];
        const float* kt = ks + t * DP + l;
#pragma unroll
        for (int i = 0; i < NPL; ++i) S[i] = fmaf(vv, kt[L * i], fmaf(-om, S[i], S[i]));
      }
    } else {
#pragma unroll 4
      for (int t = 0; t < tc; ++t) {
        const float vv = vs[t * CB + c];
        const float* kt = ks + t * DP + l;
        const float* qt = qs + t * DP + l;
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          S[i] = fmaf(vv, kt[L * i], fmaf(-om, S[i], S[i]));
          if (i & 1) a1 = fmaf(S[i], qt[L * i], a1);
          else a0 = fmaf(S[i], qt[L * i], a0);
        }
        float acc = a0 + a1;
#pragma unroll
        for (int o = 1; o < L; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (l == 0) nums[t * CB + c] = acc;
      }
      __syncthreads();
      for (int i = tid; i < tc * CB; i += THREADS) {
        const int t = i / CB, cc = i % CB;
        if (cc < vcols) y[(size_t)(row0 + first + t) * y_ld + h * V + xb * CB + cc] = nums[i];
      }
    }
  }
  if (live && (MODE != kRetFromStarts || last)) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = l + L * i;
      if (d < D) into[d] = S[i];
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
  // long segments: blocks of 16 columns walking 32 rows a batch; steps of short segments (decoding): blocks of 32
  // columns (half as many blocks fetch k and q) and batches of 4 rows
  const bool shorts = max_seg_rows > 0 && max_seg_rows <= kRetRowsShort;
#define CBIS_RET_AS(NPL, LL, CBB, TCC, MODE, Z)                                                                      \
  do {                                                                                                               \
    const size_t smem = ((size_t)2 * TCC * NPL * LL + 2 * TCC * CBB + TCC) * sizeof(float);                          \
    if (smem > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(retention_kernel<TT, NPL, LL, CBB, TCC, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                                               \
    err = launch_pdl(retention_kernel<TT, NPL, LL, CBB, TCC, MODE>, dim3((V + CBB - 1) / CBB, H, Z), dim3(CBB * LL), \
                     smem, st, (const TT*)qkv, ld, q_off, k_off, v_off, positions, freqs, rot_dims, k_scale,         \
                     one_minus_decay, state, slot_stride, seg_slot, cu_rows, y, y_ld, H, D, V, n_pieces, piece_rows, \
                     starts);                                                                                        \
  } while (0)
#define CBIS_RET(NPL, LL)                                                                                            \
  do {                                                                                                               \
    cudaError_t err = cudaSuccess;                                                                                   \
    if (n_pieces > 1) {                                                                                              \
      const int HVD = H * V * D;                                                                                     \
      CBIS_RET_AS(NPL, LL, 16, kRetRows, kRetEnds, S * n_pieces);                                                    \
      if (err != cudaSuccess) return (int)err;                                                                       \
      err = launch_pdl(retention_starts_kernel, dim3((HVD + 255) / 256, S), dim3(256), 0, st, starts,                \
                       (const float*)state, slot_stride, seg_slot, cu_rows, decay_piece, n_pieces, piece_rows,       \
                       V * D, HVD);                                                                                  \
      if (err != cudaSuccess) return (int)err;                                                                       \
      CBIS_RET_AS(NPL, LL, 16, kRetRows, kRetFromStarts, S * n_pieces);                                              \
      return (int)err;                                                                                               \
    }                                                                                                                \
    if (shorts) {                                                                                                    \
      CBIS_RET_AS(NPL, LL, 32, kRetRowsShort, kRetWhole, S);                                                         \
      return (int)err;                                                                                               \
    }                                                                                                                \
    CBIS_RET_AS(NPL, LL, 16, kRetRows, kRetWhole, S);                                                                \
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
