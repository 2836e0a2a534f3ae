// A routed mixture of gated feed-forwards.
//   * route_topk: router logits in 32-bit, a score per expert (sigmoid or softmax), the `top` largest chosen
//     (ties: the lower index), their weights the scores as they are or divided by their sum;
//   * routed_gate_up / routed_down: the chosen experts of every row, one (row, choice) pair at a time, the experts'
//     matrices streamed by warps (a row's result depends on nothing but the row: no other row of the batch and no
//     position inside it changes a sum's order).  The weight of a choice multiplies the expert's input
//     (`weight_on_input`), which for the two first products is the same as multiplying their 32-bit sums, or its output.
#include "common.cuh"

namespace cbis {

constexpr int kScoreSigmoid = 0, kScoreSoftmax = 1;

// grid (rows), 256 threads; shared: E floats.  ids [rows, top] int32, weights [rows, top] float.
template <typename TT>
__global__ void __launch_bounds__(256)
route_topk_kernel(const TT* h, int h_ld, const TT* __restrict__ router, int* ids, float* weights, int W, int E, int top,
                  int score, int renormalize, float renorm_eps, float weight_scale) {
  extern __shared__ float z[];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const TT* hr = h + (size_t)r * h_ld;
  constexpr int V = 16 / (int)sizeof(TT);      // elements of a 16-byte load
  const bool vec = W % V == 0 && !(((uintptr_t)hr | (uintptr_t)router) & 15);
  for (int e = warp; e < E; e += 8) {
    const TT* wr = router + (size_t)e * W;
    float acc = 0.f;
    if (vec) {
      float a2 = 0.f;                           // two chains of sums: the loads of a step do not wait for one another
      for (int k = lane * V; k < W; k += 32 * V) {
        TT a[V], b[V];
        *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(hr + k);
        *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(wr + k);
#pragma unroll
        for (int i = 0; i < V; i += 2) {
          acc = fmaf(to_f32(a[i]), to_f32(b[i]), acc);
          a2 = fmaf(to_f32(a[i + 1]), to_f32(b[i + 1]), a2);
        }
      }
      acc += a2;
    } else {
      for (int k = lane; k < W; k += 32) acc = fmaf(to_f32(hr[k]), to_f32(wr[k]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) z[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  float zmax = -INFINITY, denom = 1.f;
  if (score == kScoreSoftmax) {
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float d = 0.f;
    for (int e = lane; e < E; e += 32) d += expf(z[e] - zmax);
    denom = warp_sum(d);
  }
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    // the largest logit not taken yet; equal logits: the lower index
    float best = -INFINITY;
    int arg = E;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best) { best = v; arg = e; }      // within a lane indices rise, so the first of equals stays
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
    }
    if (arg >= E) arg = k < E ? k : 0;          // rows of not-a-numbers (padding): any valid expert
    const float sc = score == kScoreSoftmax ? expf(best - zmax) / denom : sigmoid_f32(best);
    total += sc;
    if (lane == 0) {
      ids[(size_t)r * top + k] = arg;
      weights[(size_t)r * top + k] = sc;
      z[arg] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0 && (renormalize || weight_scale != 1.f)) {
    const float f = renormalize ? weight_scale / (total + renorm_eps) : weight_scale;
    for (int k = 0; k < top; ++k) weights[(size_t)r * top + k] *= f;
  }
}

// grid (pairs, ceil(F / 8)), 256 threads = 8 warps, a warp per hidden column f of pair (row, choice):
//   hid[pair, f] = act(s * (Wg_e[f, :] . h[row])) * (s * (Wu_e[f, :] . h[row])),  s = weight (on input) or 1.
// gate_up: [E, 2F, W] (an expert's gate rows, then its up rows).
template <typename TT>
__global__ void __launch_bounds__(256)
routed_gate_up_kernel(const TT* h, int h_ld, const TT* __restrict__ gate_up, const int* ids, const float* weights,
                      TT* hid, int W, int F, int top, int act, int weight_on_input) {
  extern __shared__ float hs[];
  pdl_trigger();
  pdl_wait();
  const int pair = blockIdx.x, row = pair / top;
  const TT* hr = h + (size_t)row * h_ld;
  for (int k = threadIdx.x; k < W; k += 256) hs[k] = to_f32(hr[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, f = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (f >= F) return;
  const int e = ids[pair];
  const TT* wg = gate_up + ((size_t)e * 2 * F + f) * W;
  const TT* wu = wg + (size_t)F * W;
  float g = 0.f, u = 0.f;
  constexpr int V = 16 / (int)sizeof(TT);      // elements of a 16-byte load
  if (W % V == 0 && !(((uintptr_t)wg | (uintptr_t)wu) & 15)) {
    for (int k = lane * V; k < W; k += 32 * V) {
      TT a[V], b[V];
      *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(wg + k);
      *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(wu + k);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        g = fmaf(to_f32(a[i]), hs[k + i], g);
        u = fmaf(to_f32(b[i]), hs[k + i], u);
      }
    }
  } else {
    for (int k = lane; k < W; k += 32) {
      const float x = hs[k];
      g = fmaf(to_f32(wg[k]), x, g);
      u = fmaf(to_f32(wu[k]), x, u);
    }
  }
  g = warp_sum(g);
  u = warp_sum(u);
  if (lane == 0) {
    const float s = weight_on_input ? weights[pair] : 1.f;
    from_f32(hid[(size_t)pair * F + f], activate(s * g, act) * (s * u));
  }
}

// grid (rows, ceil(W / 8)), 256 threads: out[row, n] = sum over the row's choices k of
//   (weight on output ? weight : 1) * (Wd_e[n, :] . hid[row * top + k, :]),   down: [E, W, F].  out is 32-bit and is
// overwritten, or added to with `accumulate`.
template <typename TT>
__global__ void __launch_bounds__(256)
routed_down_kernel(const TT* hid, const TT* __restrict__ down, const int* ids, const float* weights, float* out,
                   int out_ld, int W, int F, int top, int weight_on_input, int accumulate) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, lane = threadIdx.x & 31, n = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (n >= W) return;
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    const int pair = row * top + k;
    const TT* wd = down + ((size_t)ids[pair] * W + n) * F;
    const TT* hp = hid + (size_t)pair * F;
    float acc = 0.f;
    constexpr int V = 16 / (int)sizeof(TT);
    if (F % V == 0 && !(((uintptr_t)wd | (uintptr_t)hp) & 15)) {
      for (int f = lane * V; f < F; f += 32 * V) {
        TT a[V], b[V];
        *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(wd + f);
        *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(hp + f);
#pragma unroll
        for (int i = 0; i < V; ++i) acc = fmaf(to_f32(a[i]), to_f32(b[i]), acc);
      }
    } else {
      for (int f = lane; f < F; f += 32) acc = fmaf(to_f32(wd[f]), to_f32(hp[f]), acc);
    }
    acc = warp_sum(acc);
    total += weight_on_input ? acc : acc * weights[pair];
  }
  if (lane == 0) {
    float* o = out + (size_t)row * out_ld + n;
    *o = accumulate ? *o + total : total;
  }
}

// ---- many rows (bfloat16): the (row, choice) pairs sorted by expert, an expert's pairs in tiles of 128 rows, each tile's
// products on the tensor cores (mma.sync m16n8k16, 32-bit sums).  A pair's result depends on its own row alone: its
// place in a tile changes no sum's order.
constexpr int kTileM = 128, kTileN = 64, kTileK = 32, kLd = kTileK + 8;   // shared rows padded to 80 bytes

// One block.  offsets [E + 1]; sorted [pairs]: the pairs expert by expert; per tile its expert, its first place in
// `sorted` and its rows; n_tiles [1].
__global__ void __launch_bounds__(1024)
routed_plan_kernel(const int* ids, int n_pairs, int E, int* offsets, int* sorted, int* tile_expert, int* tile_start,
                   int* tile_rows, int* n_tiles) {
  extern __shared__ int plan_smem[];
  int* count = plan_smem;          // E
  int* cursor = plan_smem + E;     // E
  pdl_trigger();
  pdl_wait();
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = cursor[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      for (int r = 0; r < count[e]; r += kTileM) {
        tile_expert[t] = e;
        tile_start[t] = at + r;
        tile_rows[t] = min(kTileM, count[e] - r);
        ++t;
      }
      at += count[e];
    }
    offsets[E] = at;
    *n_tiles = t;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) sorted[offsets[e] + atomicAdd(&cursor[e], 1)] = p;
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"((unsigned)__cvta_generic_to_shared(smem)));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// grid (max tiles, ceil(N / 64)), 256 threads: the eight warps own the eight 32 x 32 pieces of the 128 x 64 tile
// (with 64 x 64 tiles the blocks drew 1.35 GB through L2 in 290 us at width 2,048: the L2's rate, not the tensor cores');
// fragments come from shared memory by ldmatrix (rows 80 bytes apart: no two of a load's eight rows share a bank).
// DUAL: A = h[pair / top] (K = width), B = the expert's gate rows and up rows; out = hid[pair] = act(s g) * (s u).
// else: A = hid[pair] (K = inner), B = the expert's down matrix; y[pair] (or y[row] when top is 1) = sum (* weight).
template <bool DUAL>
__global__ void __launch_bounds__(256)
routed_tiles_kernel(const __nv_bfloat16* A, int a_ld, const __nv_bfloat16* __restrict__ Bw, const int* sorted,
                    const float* weights, const int* tile_expert, const int* tile_start, const int* tile_rows,
                    const int* n_tiles, void* out, int out_ld, int N, int K, int top, int act, int weight_on_input) {
  __shared__ __align__(16) __nv_bfloat16 As[kTileM][kLd];
  __shared__ __align__(16) __nv_bfloat16 Bs[DUAL ? 2 : 1][kTileN][kLd];
  __shared__ int pair_of[kTileM];
  pdl_trigger();
  pdl_wait();
  const int tile = blockIdx.x;
  if (tile >= *n_tiles) return;
  const int e = tile_expert[tile], start = tile_start[tile], rows = tile_rows[tile];
  const int n0 = blockIdx.y * kTileN;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < kTileM) pair_of[threadIdx.x] = threadIdx.x < rows ? sorted[start + threadIdx.x] : -1;
  __syncthreads();
  const __nv_bfloat16* B0 = Bw + (size_t)e * (DUAL ? 2 : 1) * N * K;      // [N (x2), K]
  float acc[DUAL ? 2 : 1][2][4][4];      // [gate | up][16 rows of the warp's 32][8 columns of its 32][fragment]
#pragma unroll
  for (int m = 0; m < (DUAL ? 2 : 1); ++m)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[m][mt][j][i] = 0.f;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;      // warps 4 down, 2 across
  const uint4 zero = make_uint4(0, 0, 0, 0);
  // A: 128 rows x 32 columns = 512 pieces of 16 bytes, two per thread; B: 64 x 32 = 256 pieces per matrix, one per
  // thread; the pieces of the NEXT 32 columns are fetched into registers while the tensor cores work on the ones in
  // shared memory
  constexpr int NB = DUAL ? 2 : 1;
  uint4 ra[2], rb[NB];
  const __nv_bfloat16* a_src[2];
  const int piece_k = (threadIdx.x & 3) * 8, piece_r = threadIdx.x >> 2;      // rows piece_r and piece_r + 64 of A
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int pair = pair_of[piece_r + it * 64];
    a_src[it] = pair >= 0 ? A + (size_t)(DUAL ? pair / top : pair) * a_ld : nullptr;
  }
  const __nv_bfloat16* b_src = n0 + piece_r < N ? B0 + (size_t)(n0 + piece_r) * K : nullptr;
  auto fetch = [&](int k0) {
    const int k = k0 + piece_k;
    const bool k_ok = k < K;
#pragma unroll
    for (int it = 0; it < 2; ++it) ra[it] = (a_src[it] && k_ok) ? *reinterpret_cast<const uint4*>(a_src[it] + k) : zero;
#pragma unroll
    for (int m = 0; m < NB; ++m)
      rb[m] = (b_src && k_ok) ? *reinterpret_cast<const uint4*>(b_src + (size_t)m * N * K + k) : zero;
  };
  fetch(0);
  for (int k0 = 0; k0 < K; k0 += kTileK) {
#pragma unroll
    for (int it = 0; it < 2; ++it) *reinterpret_cast<uint4*>(&As[piece_r + it * 64][piece_k]) = ra[it];
#pragma unroll
    for (int m = 0; m < NB; ++m) *reinterpret_cast<uint4*>(&Bs[m][piece_r][piece_k]) = rb[m];
    if (k0 + kTileK < K) fetch(k0 + kTileK);
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; kk += 16) {
      uint32_t a[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)      // rows (lane % 16), columns kk + 8 * (lane / 16): the four 8 x 8 quarters of A
        ldmatrix_x4(a[mt], &As[wm + mt * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int m = 0; m < NB; ++m)
#pragma unroll
        for (int jp = 0; jp < 2; ++jp) {  // two blocks of 8 columns a load: (n, k), (n, k + 8), (n + 8, k), (n + 8, k + 8)
          uint32_t b[4];
          ldmatrix_x4(b, &Bs[m][wn + jp * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
          const uint32_t b0[2] = {b[0], b[1]}, b1[2] = {b[2], b[3]};
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            mma_bf16(acc[m][mt][jp * 2], a[mt], b0);
            mma_bf16(acc[m][mt][jp * 2 + 1], a[mt], b1);
          }
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wm + mt * 16 + (lane >> 2) + half * 8;
      const int pair = pair_of[r];
      if (pair < 0) continue;
      const float w = weights[pair];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int n = n0 + wn + j * 8 + (lane & 3) * 2 + i;
          if (n >= N) continue;
          const float v0 = acc[0][mt][j][half * 2 + i];
          if (DUAL) {
            const float s = weight_on_input ? w : 1.f;
            from_f32(static_cast<__nv_bfloat16*>(out)[(size_t)pair * out_ld + n],
                     activate(s * v0, act) * (s * acc[DUAL ? 1 : 0][mt][j][half * 2 + i]));
          } else {
            static_cast<float*>(out)[(size_t)pair * out_ld + n] = weight_on_input ? v0 : w * v0;
          }
        }
    }
}

// out[row, n] (+)= y[row * top + 0, n] + y[row * top + 1, n] + ..., in that order; 32-bit.
__global__ void routed_combine_kernel(const float* y, float* out, int out_ld, int rows, int W, int top, int accumulate) {
  pdl_trigger();
  pdl_wait();
  const size_t total = (size_t)rows * W;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / W;
    const int n = (int)(i % W);
    float v = 0.f;
    for (int k = 0; k < top; ++k) v += y[(r * top + k) * W + n];
    float* o = out + r * out_ld + n;
    *o = accumulate ? *o + v : v;
  }
}

}  // namespace cbis

using namespace cbis;

CBIS_EXPORT int cbis_routed_tile_rows() { return kTileM; }

// ints of scratch the plan needs: offsets (E + 1), sorted (pairs), three tables of max_tiles, n_tiles (1)
CBIS_EXPORT long long cbis_routed_plan_ints(int pairs, int E) {
  const long long max_tiles = (pairs + kTileM - 1) / kTileM + E;
  return (long long)E + 1 + pairs + 3 * max_tiles + 1;
}

// The whole routed feed-forward for many rows of bfloat16: plan, gate/up tiles, down tiles, and (top > 1) the sum of a
// row's choices.  plan: cbis_routed_plan_ints ints; hid [pairs, F] bfloat16; y [pairs, W] 32-bit (unused when top is 1);
// out [rows, W] 32-bit, overwritten, or added to with `accumulate`.
CBIS_EXPORT int cbis_routed_tiles(const void* h, int h_ld, const void* gate_up, const void* down, const int* ids,
                                  const float* weights, int* plan, void* hid, float* y, float* out, int out_ld, int rows,
                                  int W, int F, int E, int top, int act, int weight_on_input, int accumulate,
                                  void* stream) {
  if (rows <= 0) return CBIS_OK;
  if (W <= 0 || F <= 0 || E <= 0 || top <= 0) return CBIS_ERR_BAD_SIZE;
  if (W % 8 || F % 8 || h_ld % 8) return CBIS_ERR_ALIGNMENT;
  if (((uintptr_t)h | (uintptr_t)gate_up | (uintptr_t)down | (uintptr_t)hid) & 15) return CBIS_ERR_ALIGNMENT;
  if (E > 4096) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const int pairs = rows * top;
  const int max_tiles = (pairs + kTileM - 1) / kTileM + E;
  int* offsets = plan;
  int* sorted = offsets + E + 1;
  int* tile_expert = sorted + pairs;
  int* tile_start = tile_expert + max_tiles;
  int* tile_rows = tile_start + max_tiles;
  int* n_tiles = tile_rows + max_tiles;
  cudaError_t err = launch_pdl(routed_plan_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), st, ids, pairs, E,
                               offsets, sorted, tile_expert, tile_start, tile_rows, n_tiles);
  if (err != cudaSuccess) return (int)err;
  typedef const __nv_bfloat16* bp;
  err = launch_pdl(routed_tiles_kernel<true>, dim3(max_tiles, (F + kTileN - 1) / kTileN), dim3(256), 0, st, (bp)h, h_ld,
                   (bp)gate_up, (const int*)sorted, weights, (const int*)tile_expert, (const int*)tile_start,
                   (const int*)tile_rows, (const int*)n_tiles, hid, F, F, W, top, act, weight_on_input);
  if (err != cudaSuccess) return (int)err;
  const bool direct = top == 1 && !accumulate;
  err = launch_pdl(routed_tiles_kernel<false>, dim3(max_tiles, (W + kTileN - 1) / kTileN), dim3(256), 0, st, (bp)hid, F,
                   (bp)down, (const int*)sorted, weights, (const int*)tile_expert, (const int*)tile_start,
                   (const int*)tile_rows, (const int*)n_tiles, (void*)(direct ? out : y), direct ? out_ld : W, W, F, top,
                   act, weight_on_input);
  if (err != cudaSuccess || direct) return (int)err;
  const size_t total = (size_t)rows * W;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return (int)launch_pdl(routed_combine_kernel, dim3((int)blocks), dim3(256), 0, st, (const float*)y, out, out_ld, rows, W,
                         top, accumulate);
}

CBIS_EXPORT int cbis_route_topk(const void* h, int h_ld, const void* router, int* ids, float* weights, int rows, int W,
                                int E, int top, int score, int renormalize, int dtype, void* stream, float renorm_eps,
                                float weight_scale) {
  if (rows <= 0) return CBIS_OK;
  if (W <= 0 || E <= 0 || top <= 0 || top > E || (score != kScoreSigmoid && score != kScoreSoftmax)) return CBIS_ERR_BAD_SIZE;
  if (E > 8192) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)E * sizeof(float);
  if (dtype == CBIS_F32)
    return (int)launch_pdl(route_topk_kernel<float>, dim3(rows), dim3(256), smem, st, (const float*)h, h_ld,
                           (const float*)router, ids, weights, W, E, top, score, renormalize, renorm_eps, weight_scale);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(route_topk_kernel<__nv_bfloat16>, dim3(rows), dim3(256), smem, st, (const __nv_bfloat16*)h, h_ld,
                           (const __nv_bfloat16*)router, ids, weights, W, E, top, score, renormalize, renorm_eps,
                           weight_scale);
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_routed_gate_up(const void* h, int h_ld, const void* gate_up, const int* ids, const float* weights,
                                    void* hid, int rows, int W, int F, int top, int act, int weight_on_input, int dtype,
                                    void* stream) {
  if (rows <= 0) return CBIS_OK;
  if (W <= 0 || F <= 0 || top <= 0) return CBIS_ERR_BAD_SIZE;
  if (W > 12288 || F > 8 * 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid(rows * top, (F + 7) / 8);
  const size_t smem = (size_t)W * sizeof(float);
  if (dtype == CBIS_F32)
    return (int)launch_pdl(routed_gate_up_kernel<float>, grid, dim3(256), smem, st, (const float*)h, h_ld,
                           (const float*)gate_up, ids, weights, (float*)hid, W, F, top, act, weight_on_input);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(routed_gate_up_kernel<__nv_bfloat16>, grid, dim3(256), smem, st, (const __nv_bfloat16*)h, h_ld,
                           (const __nv_bfloat16*)gate_up, ids, weights, (__nv_bfloat16*)hid, W, F, top, act,
                           weight_on_input);
  return CBIS_ERR_BAD_DTYPE;
}

CBIS_EXPORT int cbis_routed_down(const void* hid, const void* down, const int* ids, const float* weights, float* out,
                                 int out_ld, int rows, int W, int F, int top, int weight_on_input, int accumulate,
                                 int dtype, void* stream) {
  if (rows <= 0) return CBIS_OK;
  if (W <= 0 || F <= 0 || top <= 0) return CBIS_ERR_BAD_SIZE;
  if (W > 8 * 65535) return CBIS_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid(rows, (W + 7) / 8);
  if (dtype == CBIS_F32)
    return (int)launch_pdl(routed_down_kernel<float>, grid, dim3(256), 0, st, (const float*)hid, (const float*)down, ids,
                           weights, out, out_ld, W, F, top, weight_on_input, accumulate);
  if (dtype == CBIS_BF16)
    return (int)launch_pdl(routed_down_kernel<__nv_bfloat16>, grid, dim3(256), 0, st, (const __nv_bfloat16*)hid,
                           (const __nv_bfloat16*)down, ids, weights, out, out_ld, W, F, top, weight_on_input, accumulate);
  return CBIS_ERR_BAD_DTYPE;
}
