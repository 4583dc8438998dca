// A routed feed-forward (mixture of experts) in five launches, none of which needs a number on the host:
//   moe_route     scores s = sigmoid(logits) (or softmax over the experts); groups of neighbouring experts scored by their two
//                 best; the best `keep` groups stay; the `top` best experts among them; weights s / (sum s + 1e-20) * scale
//                 (float32).  With a correction vector c the comparisons use s + c, the weights s.
//   moe_sort      the (row, choice) pairs ordered by expert: offsets of every expert's pairs and of its row tiles
//   moe_gemm 0    z[i] = act(W_gate[e] h[row]) * (W_up[e] h[row])      for the sorted pairs i (a tile = 32 pairs of one expert)
//   moe_gemm 1    y[pair] = W_down[e] z[i]                             float32, back at the pair's own place
//   moe_combine   x[row] += sum_j weight[row, j] * y[row * top + j]    ascending j, float32; a shared expert's rows (float32), times
//                 the sigmoid of a gate logit a row where one is given, join the sum behind the chosen experts' 
// A pair's sums run over k in ascending order with one accumulator, so its result does not depend on which other
// rows share its tile, nor on the order in which the sort placed the pairs of an expert.
//
// Two more roads, chosen by the caller from the step's size alone:
//   many pairs, bfloat16   moe_sort_tiles lays every expert's pairs out from a multiple of 256 rows on and names each row
//                          tile's expert; moe_gather_rows copies the rows of h to their places; the two products run on
//                          the tcgen05 kernel (gemm_tcgen05_pair_grouped); moe_combine reads y through the pairs' places
//   few pairs, bfloat16    moe_few: a warp computes one output feature for up to 8 pairs of an expert, streaming the
//                          feature's weights with 16-byte loads (a decode step reads every touched expert once)
#include "common.cuh"

namespace {
constexpr int MOE_MAX_EXPERTS = 1024;
constexpr int BM = 32, BN = 64, BK = 16;

// The pairs of idx [P] ordered by expert, by the threads of one block (cnt, off: shared memory of MOE_MAX_EXPERTS (+ 1) ints).
__device__ __forceinline__ void moe_sort_block(const int* idx, int P, int E, int* offsets, int* tiles, int* perm, int* cnt, int* off) {
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cnt[idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, t = 0;
    for (int e = 0; e < E; e++) {
      off[e] = o; offsets[e] = o; tiles[e] = t;
      o += cnt[e];
      t += (cnt[e] + BM - 1) / BM;
    }
    off[E] = o; offsets[E] = o; tiles[E] = t;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = idx[p];
    perm[off[e] + atomicAdd(&cnt[e], 1)] = p;
  }
}

// One thread a row.  With at most ROUTE_SMEM_EXPERTS experts the row's scores live in shared memory (a decode step's
// few rows would otherwise walk dependent loads from global memory); with more they stay in the caller's buffer.
constexpr int ROUTE_THREADS = 64, ROUTE_SMEM_EXPERTS = 128;
__device__ __forceinline__ void moe_route_row(float* scores, float* local, int row, int E, int ld, int top, int groups, int keep, float scale,
                                              int softmax, const float* corr, int* idx, float* wgt);
__global__ void __launch_bounds__(ROUTE_THREADS)
k_moe_route(float* __restrict__ scores, int T, int E, int ld, int top, int groups, int keep, float scale, int softmax,
            const float* __restrict__ corr, int* __restrict__ idx,
            float* __restrict__ wgt, int* __restrict__ offsets, int* __restrict__ tiles, int* __restrict__ perm) {
  cima_pdl_wait();
  cima_pdl_trigger();        // the next kernel may be set up while this one runs (it waits for this one's end itself)
  __shared__ float local[ROUTE_THREADS * (ROUTE_SMEM_EXPERTS + 1)];
  __shared__ int cnt[MOE_MAX_EXPERTS];
  __shared__ int off[MOE_MAX_EXPERTS + 1];
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row < T) moe_route_row(scores, local, row, E, ld, top, groups, keep, scale, softmax, corr, idx, wgt);
  if (offsets) {             // a step of one block's rows: the pairs are ordered by expert here, which saves moe_sort's launch
    __syncthreads();
    moe_sort_block(idx, T * top, E, offsets, tiles, perm, cnt, off);
  }
}

__device__ __forceinline__ void moe_route_row(float* scores, float* local, int row, int E, int ld, int top, int groups, int keep, float scale,
                                              int softmax, const float* corr, int* idx, float* wgt) {
  float* s = E <= ROUTE_SMEM_EXPERTS ? local + threadIdx.x * (E + 1) : scores + (size_t)row * ld;
  const float* z = scores + (size_t)row * ld;
  float zmax = -INFINITY;
  if (softmax)
    for (int e = 0; e < E; e++) zmax = fmaxf(zmax, z[e]);
  float den = 0.f;
  for (int e0 = 0; e0 < E; e0 += 8) {                     // eight logits requested before any is waited for
    float t[8];
#pragma unroll
    for (int j = 0; j < 8; j++) t[j] = e0 + j < E ? z[e0 + j] : 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++)
      if (e0 + j < E) {
        const float v = softmax ? expf(t[j] - zmax) : 1.0f / (1.0f + expf(-t[j]));
        s[e0 + j] = v;
        den += v;
      }
  }
  if (softmax) {
    const float inv = 1.0f / den;
    for (int e = 0; e < E; e++) s[e] *= inv;
  }
  // an expert is compared by s + its correction and weighted by s; a taken one is marked with -inf
  const int per = E / groups;
  unsigned long long kept = ~0ull;
  if (keep < groups) {
    kept = 0ull;
    for (int c = 0; c < keep; c++) {
      int best = -1;
      float bs = -INFINITY;
      for (int gi = 0; gi < groups; gi++) {
        if ((kept >> gi) & 1ull) continue;
        float a1 = -INFINITY, a2 = -INFINITY;              // the group's two largest scores
        for (int e = gi * per; e < (gi + 1) * per; e++) {
          const float v = s[e] + (corr ? corr[e] : 0.f);
          if (v > a1) { a2 = a1; a1 = v; } else if (v > a2) a2 = v;
        }
        const float sc = per >= 2 ? a1 + a2 : a1;
        if (sc > bs || best < 0) { bs = sc; best = gi; }
      }
      kept |= 1ull << best;
    }
  }
  float sum = 0.f;
  for (int c = 0; c < top; c++) {
    int best = -1;
    float bs = -INFINITY;
    for (int gi = 0; gi < groups; gi++) {
      if (!((kept >> gi) & 1ull)) continue;
      for (int e = gi * per; e < (gi + 1) * per; e++) {
        const float raw = s[e];
        if (raw == -INFINITY) continue;
        const float v = raw + (corr ? corr[e] : 0.f);
        if (v > bs || best < 0) { bs = v; best = e; }
      }
    }
    const float w = s[best];
    idx[(size_t)row * top + c] = best;
    wgt[(size_t)row * top + c] = w;
    sum += w;
    s[best] = -INFINITY;                                   // taken
  }
  const float f = scale / (sum + 1e-20f);
  for (int c = 0; c < top; c++) wgt[(size_t)row * top + c] *= f;
}

// offsets [E + 1]: first sorted pair of every expert; tiles [E + 1]: first row tile of every expert; perm [P]: the
// pair at every sorted place.  One block.
__global__ void __launch_bounds__(1024)
k_moe_sort(const int* __restrict__ idx, int P, int E, int* __restrict__ offsets, int* __restrict__ tiles, int* __restrict__ perm) {
  cima_pdl_wait();
  cima_pdl_trigger();        // the next kernel may be set up while this one runs (it waits for this one's end itself)
  __shared__ int cnt[MOE_MAX_EXPERTS];
  __shared__ int off[MOE_MAX_EXPERTS + 1];
  moe_sort_block(idx, P, E, offsets, tiles, perm, cnt, off);
}

// MODE 0: A = h [T, K] gathered by row = perm[i] / top; W = [E, 2 N, K] (gate rows, then up rows); out z [P, N] (TA) at i.
// MODE 1: A = z [P, K] at i; W = [E, N, K]; out y [P, N] float32 at perm[i].
template <typename TA, typename TW, int MODE>
__global__ void __launch_bounds__(256)
k_moe_gemm(const TA* __restrict__ A, int lda, const TW* __restrict__ W, void* __restrict__ out, const int* __restrict__ offsets,
           const int* __restrict__ tiles, const int* __restrict__ perm, int E, int top, int N, int K, int act, float limit) {
  cima_pdl_wait();
  __shared__ float As[BK][BM + 1];
  __shared__ float Bs[MODE == 0 ? 2 : 1][BK][BN + 1];
  __shared__ int s_row[BM];
  __shared__ int s_e, s_i0, s_n;
  if (threadIdx.x == 0) {
    const int tile = blockIdx.x;
    int e = -1;
    if (tile < tiles[E]) {
      // the expert whose tiles hold this one (tiles is ascending; experts without pairs own none)
      int lo = 0, hi = E - 1;
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (tiles[mid] <= tile) lo = mid; else hi = mid - 1; }
      e = lo;
      while (tiles[e + 1] <= tile) e++;                     // (skips experts without tiles that share the start)
      s_i0 = offsets[e] + (tile - tiles[e]) * BM;
      s_n = min(BM, offsets[e + 1] - s_i0);
    }
    s_e = e;
  }
  __syncthreads();
  const int e = s_e;
  if (e < 0) return;
  const int i0 = s_i0, nrows = s_n;
  if (threadIdx.x < BM) {
    const int r = threadIdx.x;
    s_row[r] = r < nrows ? (MODE == 0 ? perm[i0 + r] / top : i0 + r) : -1;
  }
  __syncthreads();
  const int n0 = blockIdx.y * BN;
  const TW* Wg = W + (size_t)e * (MODE == 0 ? 2 : 1) * N * K;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // tx: 4 columns each, ty: 2 rows each
  float acc[2][4] = {}, acc2[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int t = threadIdx.x; t < BM * BK; t += 256) {
      const int r = t / BK, kk = t - r * BK;
      const int src = s_row[r];
      As[kk][r] = (src >= 0 && k0 + kk < K) ? cima_to_f32<TA>(A[(size_t)src * lda + k0 + kk]) : 0.f;
    }
    for (int t = threadIdx.x; t < BN * BK; t += 256) {
      const int c = t / BK, kk = t - c * BK;
      const bool ok = n0 + c < N && k0 + kk < K;
      Bs[0][kk][c] = ok ? cima_to_f32<TW>(Wg[(size_t)(n0 + c) * K + k0 + kk]) : 0.f;
      if (MODE == 0) Bs[1][kk][c] = ok ? cima_to_f32<TW>(Wg[(size_t)(N + n0 + c) * K + k0 + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float b = Bs[0][kk][tx * 4 + j];
        acc[0][j] = fmaf(a0, b, acc[0][j]);
        acc[1][j] = fmaf(a1, b, acc[1][j]);
        if (MODE == 0) {
          const float b2 = Bs[1][kk][tx * 4 + j];
          acc2[0][j] = fmaf(a0, b2, acc2[0][j]);
          acc2[1][j] = fmaf(a1, b2, acc2[1][j]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int r = ty * 2 + i;
    if (r >= nrows) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int c = n0 + tx * 4 + j;
      if (c >= N) continue;
      if (MODE == 0) {
        // the gate is rounded to the activations' dtype before its activation, as a stored projection would be
        const float gt = cima_to_f32<TA>(cima_from_f32<TA>(acc[i][j])), up = cima_to_f32<TA>(cima_from_f32<TA>(acc2[i][j]));
        reinterpret_cast<TA*>(out)[(size_t)(i0 + r) * N + c] = cima_from_f32<TA>(cima_gated(gt, up, act, limit));
      } else {
        reinterpret_cast<float*>(out)[(size_t)perm[i0 + r] * N + c] = acc[i][j];
      }
    }
  }
}

// pos: the row of y that holds pair (row, j), or null where y is kept by pair
__global__ void __launch_bounds__(256)
k_moe_combine(const float* __restrict__ y, const float* __restrict__ wgt, const int* __restrict__ pos, float* __restrict__ x,
              int top, int H, int assign, const float* __restrict__ shared, const float* __restrict__ gate, int ldg) {
  cima_pdl_wait();
  cima_pdl_trigger();        // the next kernel may be set up while this one runs (it waits for this one's end itself)
  const size_t row = blockIdx.x;
  const float sg = shared ? (gate ? 1.0f / (1.0f + expf(-gate[row * (size_t)ldg])) : 1.0f) : 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float s = 0.f;
    for (int j = 0; j < top; j++) {
      const size_t p = row * top + j;
      s = fmaf(wgt[p], y[(pos ? (size_t)pos[p] : p) * H + c], s);
    }
    if (shared) s = fmaf(sg, shared[row * H + c], s);
    x[row * H + c] = assign ? s : x[row * H + c] + s;
  }
}

// The same for rows whose width is a multiple of 4 and at most COMBINE_TOP choices: four columns a thread, the choices'
// weights and places fetched once a row, and the rows of all choices requested before the first is used.  The sum runs
// over j in the same ascending order.
constexpr int COMBINE_TOP = 8;
__global__ void __launch_bounds__(128)
k_moe_combine4(const float* __restrict__ y, const float* __restrict__ wgt, const int* __restrict__ pos, float* __restrict__ x,
               int top, int H4, int assign, const float* __restrict__ shared, const float* __restrict__ gate, int ldg) {
  cima_pdl_wait();
  cima_pdl_trigger();
  const size_t row = blockIdx.x;
  float w[COMBINE_TOP];
  const float4* src[COMBINE_TOP];
#pragma unroll
  for (int j = 0; j < COMBINE_TOP; j++) {
    const size_t p = row * top + (j < top ? j : 0);
    w[j] = j < top ? wgt[p] : 0.f;
    src[j] = reinterpret_cast<const float4*>(y) + (pos ? (size_t)pos[p] : p) * H4;
  }
  const float sg = shared ? (gate ? 1.0f / (1.0f + expf(-gate[row * (size_t)ldg])) : 1.0f) : 0.f;
  const float4* sh = shared ? reinterpret_cast<const float4*>(shared) + row * H4 : nullptr;
  float4* xr = reinterpret_cast<float4*>(x) + row * H4;
  // (a block takes 128 groups of four columns: a decode step's few rows are spread over many blocks)
  for (int g = blockIdx.y * blockDim.x + threadIdx.x; g < H4; g += gridDim.y * blockDim.x) {
    float4 v[COMBINE_TOP];
#pragma unroll
    for (int j = 0; j < COMBINE_TOP; j++) v[j] = j < top ? src[j][g] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 sv = sh ? sh[g] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 xo = assign ? make_float4(0.f, 0.f, 0.f, 0.f) : xr[g];
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < COMBINE_TOP; j++)
      if (j < top) { s.x = fmaf(w[j], v[j].x, s.x); s.y = fmaf(w[j], v[j].y, s.y); s.z = fmaf(w[j], v[j].z, s.z); s.w = fmaf(w[j], v[j].w, s.w); }
    if (sh) { s.x = fmaf(sg, sv.x, s.x); s.y = fmaf(sg, sv.y, s.y); s.z = fmaf(sg, sv.z, s.z); s.w = fmaf(sg, sv.w, s.w); }
    xr[g] = assign ? s : make_float4(xo.x + s.x, xo.y + s.y, xo.z + s.z, xo.w + s.w);
  }
}

// Every expert's pairs from a multiple of `tile` rows on: pos [P] the place of every pair, tile_expert [n_tiles] the
// expert of every row tile (-1 beyond the last).  One block.
__global__ void __launch_bounds__(1024)
k_moe_sort_tiles(const int* __restrict__ idx, int P, int E, int tile, int n_tiles, int* __restrict__ tile_expert, int* __restrict__ pos) {
  cima_pdl_wait();
  cima_pdl_trigger();        // the next kernel may be set up while this one runs (it waits for this one's end itself)
  __shared__ int cnt[MOE_MAX_EXPERTS];
  __shared__ int off[MOE_MAX_EXPERTS + 1];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&cnt[idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int e = 0; e < E; e++) { off[e] = t; t += (cnt[e] + tile - 1) / tile; }
    off[E] = t;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) {
    int e = -1;
    if (t < off[E]) {
      int lo = 0, hi = E - 1;
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (off[mid] <= t) lo = mid; else hi = mid - 1; }
      e = lo;
      while (off[e + 1] <= t) e++;
    }
    tile_expert[t] = e;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int e = idx[p];
    pos[p] = off[e] * tile + atomicAdd(&cnt[e], 1);
  }
}

// dst[pos[p]] = src[p / top]: rows of K values, 16 bytes a thread
__global__ void __launch_bounds__(256)
k_moe_gather_rows(const uint4* __restrict__ src, const int* __restrict__ pos, uint4* __restrict__ dst, int top, int vecs) {
  cima_pdl_wait();
  cima_pdl_trigger();        // the next kernel may be set up while this one runs (it waits for this one's end itself)
  const size_t p = blockIdx.x;
  const uint4* s = src + (p / top) * vecs;
  uint4* d = dst + (size_t)pos[p] * vecs;
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) d[v] = s[v];
}

// Few pairs (a decode step).  Block (x = tile of 32 pairs of one expert as moe_sort laid them out, y = 8 or 16 output
// features): warp w owns feature n0 + w (and n0 + w + 8); its lanes stride the features' weights by 16 bytes and hold the sums
// of up to 8 pairs at a time; a fixed shuffle tree adds the lanes.  MODE as in k_moe_gemm.
constexpr int FEW_PAIRS = 8;
constexpr int FEW_ROWS = 2;          // rows of weights a warp streams at once (4 measured the same: 0.663 against 0.659 ms a step)
template <int MODE>
__global__ void __launch_bounds__(256)
k_moe_few(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, void* __restrict__ out,
          const int* __restrict__ offsets, const int* __restrict__ tiles, const int* __restrict__ perm, int E, int top, int N,
          int K, int act, float limit) {
  cima_pdl_wait();
  __shared__ int s_row[BM];
  __shared__ int s_e, s_i0, s_n;
  if (threadIdx.x == 0) {
    const int tile = blockIdx.x;
    int e = -1;
    if (tile < tiles[E]) {
      int lo = 0, hi = E - 1;
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (tiles[mid] <= tile) lo = mid; else hi = mid - 1; }
      e = lo;
      while (tiles[e + 1] <= tile) e++;
      s_i0 = offsets[e] + (tile - tiles[e]) * BM;
      s_n = min(BM, offsets[e + 1] - s_i0);
    }
    s_e = e;
  }
  __syncthreads();
  const int e = s_e;
  if (e < 0) return;
  const int i0 = s_i0, nrows = s_n;
  const int tid = (int)threadIdx.x;
  if (tid < BM) s_row[tid] = tid < nrows ? (MODE == 0 ? perm[i0 + tid] / top : i0 + tid) : -1;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // A warp streams FEW_ROWS rows of weights at once, so that enough loads are in flight: a feature's gate and up rows
  // (MODE 0) or the rows of features n and n + 8 (MODE 1); with four, two and four features.  With one row a warp the down
  // product stood at 0.4 of the bandwidth (a decode step of the 1.5B shape at batch 8 took 0.72 ms, with two 0.66 ms).
  constexpr int FEATS = MODE == 0 ? FEW_ROWS / 2 : FEW_ROWS;          // features a warp computes
  const int n = blockIdx.y * (8 * FEATS) + warp;
  if (n >= N) return;
  const __nv_bfloat16* wrow[FEW_ROWS];
  bool valid[FEATS];
#pragma unroll
  for (int f = 0; f < FEATS; f++) {
    valid[f] = n + 8 * f < N;
    const int nf = valid[f] ? n + 8 * f : n;
    if (MODE == 0) {
      wrow[2 * f] = W + ((size_t)e * 2 * N + nf) * K;
      wrow[2 * f + 1] = wrow[2 * f] + (size_t)N * K;
    } else {
      wrow[f] = W + ((size_t)e * N + nf) * K;
    }
  }
  for (int r0 = 0; r0 < nrows; r0 += FEW_PAIRS) {
    float acc[FEW_ROWS][FEW_PAIRS];
#pragma unroll
    for (int j = 0; j < FEW_ROWS; j++)
#pragma unroll
      for (int r = 0; r < FEW_PAIRS; r++) acc[j][r] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
      uint4 w4[FEW_ROWS];
#pragma unroll
      for (int j = 0; j < FEW_ROWS; j++) w4[j] = *reinterpret_cast<const uint4*>(wrow[j] + k);
#pragma unroll
      for (int r = 0; r < FEW_PAIRS; r++) {
        if (r0 + r >= nrows) break;
        const uint4 a4 = *reinterpret_cast<const uint4*>(A + (size_t)s_row[r0 + r] * lda + k);
        const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a4);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const float2 av = __bfloat1622float2(ap[q]);
#pragma unroll
          for (int j = 0; j < FEW_ROWS; j++) {
            const float2 wv = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(&w4[j])[q]);
            acc[j][r] = fmaf(av.x, wv.x, acc[j][r]);
            acc[j][r] = fmaf(av.y, wv.y, acc[j][r]);
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < FEW_PAIRS; r++) {
#pragma unroll
      for (int j = 0; j < FEW_ROWS; j++)
        for (int o = 16; o > 0; o >>= 1) acc[j][r] += __shfl_xor_sync(0xffffffffu, acc[j][r], o);
      if (lane == 0 && r0 + r < nrows) {
#pragma unroll
        for (int f = 0; f < FEATS; f++) {
          if (!valid[f]) continue;
          if (MODE == 0) {
            // gate and up are rounded to bfloat16 before the activation, as stored projections would be
            const float gt = __bfloat162float(__float2bfloat16_rn(acc[2 * f][r])), uv = __bfloat162float(__float2bfloat16_rn(acc[2 * f + 1][r]));
            reinterpret_cast<__nv_bfloat16*>(out)[(size_t)(i0 + r0 + r) * N + n + 8 * f] = __float2bfloat16_rn(cima_gated(gt, uv, act, limit));
          } else {
            reinterpret_cast<float*>(out)[(size_t)perm[i0 + r0 + r] * N + n + 8 * f] = acc[f][r];
          }
        }
      }
    }
  }
}
}  // namespace

// scores [T, E] float32: the router's logits on entry, scratch afterwards.  idx [T, top] int32, wgt [T, top] float32.
// offsets, tiles, perm: null, or (at most 64 rows) the outputs of moe_sort, made by the same launch.
extern "C" int cima_moe_route(float* scores, int T, int E, int ld, int top, int groups, int keep, float scale, int softmax,
                              const float* correction, int* idx, float* wgt,
                              int* offsets, int* tiles, int* perm, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (ld < E) return cima_fail(CIMA_E_SIZE, "moe_route: rows of %d scores hold no %d experts", ld, E);
  if (E <= 0 || E > MOE_MAX_EXPERTS || groups <= 0 || groups > 64 || E % groups || keep <= 0 || keep > groups)
    return cima_fail(CIMA_E_SIZE, "moe_route: %d experts in %d groups of which %d stay are not accepted (at most %d experts in at most 64 equal groups)", E, groups, keep, MOE_MAX_EXPERTS);
  if (top <= 0 || top > keep * (E / groups)) return cima_fail(CIMA_E_SIZE, "moe_route: %d choices among %d experts that stay", top, keep * (E / groups));
  if ((offsets || tiles || perm) && (!offsets || !tiles || !perm || T > ROUTE_THREADS))
    return cima_fail(CIMA_E_ARG, "moe_route: ordering the pairs here takes offsets, tiles and perm and at most %d rows (%d given)", ROUTE_THREADS, T);
  int rc = cima_launch(k_moe_route, dim3((T + ROUTE_THREADS - 1) / ROUTE_THREADS), dim3(ROUTE_THREADS), (size_t)0, stream, 1, scores, T, E, ld, top, groups, keep, scale, softmax, correction, idx, wgt, offsets, tiles, perm);
  return rc ? rc : cima_launch_result();
}

extern "C" int cima_moe_sort(const int* idx, int P, int E, int* offsets, int* tiles, int* perm, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (E <= 0 || E > MOE_MAX_EXPERTS) return cima_fail(CIMA_E_SIZE, "moe_sort: %d experts (at most %d)", E, MOE_MAX_EXPERTS);
  int rc = cima_launch(k_moe_sort, dim3(1), dim3(1024), (size_t)0, stream, 1, idx, P, E, offsets, tiles, perm);
  return rc ? rc : cima_launch_result();
}

// mode 0: a [T, lda] (adtype), w [E, 2 N, K] (wdtype), out [P, N] (adtype); mode 1: a [P, lda], w [E, N, K], out [P, N] float32.
extern "C" int cima_moe_gemm(const void* a, int adtype, int lda, const void* w, int wdtype, void* out, const int* offsets,
                             const int* tiles, const int* perm, int P, int E, int top, int N, int K, int mode, int act, float limit,
                             cudaStream_t stream) {
  if (P <= 0) return 0;
  if (N <= 0 || K <= 0 || E <= 0 || top <= 0) return cima_fail(CIMA_E_SIZE, "moe_gemm: sizes must be positive");
  if (mode != 0 && mode != 1) return cima_fail(CIMA_E_ARG, "moe_gemm: mode %d is neither 0 (gate | up) nor 1 (down)", mode);
  if (act < 0 || act >= CIMA_GATED_COUNT) return cima_fail(CIMA_E_ARG, "moe_gemm: activation code %d is unknown", act);
  const dim3 grid((unsigned)((P + BM - 1) / BM + E), (unsigned)((N + BN - 1) / BN));
  if (grid.y > 65535) return cima_fail(CIMA_E_SIZE, "moe_gemm: %d outputs exceed one launch", N);
  int rc;
#define RUN(TA, TW, M) rc = cima_launch(k_moe_gemm<TA, TW, M>, grid, dim3(256), (size_t)0, stream, 1, (const TA*)a, lda, (const TW*)w, out, offsets, tiles, perm, E, top, N, K, act, limit)
  if (adtype == CIMA_F32 && wdtype == CIMA_F32) { if (mode == 0) RUN(float, float, 0); else RUN(float, float, 1); }
  else if (adtype == CIMA_BF16 && wdtype == CIMA_BF16) { if (mode == 0) RUN(__nv_bfloat16, __nv_bfloat16, 0); else RUN(__nv_bfloat16, __nv_bfloat16, 1); }
  else if (adtype == CIMA_BF16 && wdtype == CIMA_F32) { if (mode == 0) RUN(__nv_bfloat16, float, 0); else RUN(__nv_bfloat16, float, 1); }
  else return cima_fail(CIMA_E_DTYPE, "moe_gemm: activations of dtype %d with weights of dtype %d are not accepted", adtype, wdtype);
#undef RUN
  return rc ? rc : cima_launch_result();
}

// y [pairs or places, H] float32; pos [T * top] the row of y of every pair, or null where y is kept by pair
// shared (may be null): [T, H] float32 rows added behind the experts', each row times sigmoid(gate[row * ldg]) where gate is given
extern "C" int cima_moe_combine(const float* y, const float* wgt, const int* pos, float* x, int T, int top, int H, int assign,
                                const float* shared, const float* gate, int ldg, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (top <= COMBINE_TOP && H % 4 == 0 && (((uintptr_t)y | (uintptr_t)x | (uintptr_t)shared) & 15) == 0) {
    const unsigned parts = (unsigned)((H / 4 + 127) / 128);
    int rc4 = cima_launch(k_moe_combine4, dim3(T, parts > 65535 ? 65535 : parts), dim3(128), (size_t)0, stream, 1, y, wgt, pos, x, top, H / 4, assign, shared, gate, ldg);
    return rc4 ? rc4 : cima_launch_result();
  }
  int rc = cima_launch(k_moe_combine, dim3(T), dim3(256), (size_t)0, stream, 1, y, wgt, pos, x, top, H, assign, shared, gate, ldg);
  return rc ? rc : cima_launch_result();
}

// tile_expert [n_tiles] and pos [P] as k_moe_sort_tiles describes; n_tiles >= ceil(P / tile) + E holds every layout.
extern "C" int cima_moe_sort_tiles(const int* idx, int P, int E, int tile, int n_tiles, int* tile_expert, int* pos, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (E <= 0 || E > MOE_MAX_EXPERTS || tile <= 0 || n_tiles < (P + tile - 1) / tile)
    return cima_fail(CIMA_E_SIZE, "moe_sort_tiles: %d experts (at most %d), tiles of %d rows, %d tiles for %d pairs", E, MOE_MAX_EXPERTS, tile, n_tiles, P);
  int rc = cima_launch(k_moe_sort_tiles, dim3(1), dim3(1024), (size_t)0, stream, 1, idx, P, E, tile, n_tiles, tile_expert, pos);
  return rc ? rc : cima_launch_result();
}

// dst[pos[p]] = src[p / top] for the P pairs: rows of `row_bytes` bytes (a multiple of 16, both 16-byte aligned)
extern "C" int cima_moe_gather_rows(const void* src, const int* pos, void* dst, int P, int top, int row_bytes, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (row_bytes <= 0 || row_bytes % 16 || (((uintptr_t)src | (uintptr_t)dst) & 15))
    return cima_fail(CIMA_E_ARG, "moe_gather_rows: rows of %d bytes must be multiples of 16 bytes at 16-byte aligned addresses", row_bytes);
  int rc = cima_launch(k_moe_gather_rows, dim3(P), dim3(256), (size_t)0, stream, 1, (const uint4*)src, pos, (uint4*)dst, top, row_bytes / 16);
  return rc ? rc : cima_launch_result();
}

// The products of moe_gemm for few pairs, bfloat16 activations and weights, K a multiple of 8, 16-byte aligned rows.
extern "C" int cima_moe_few(const void* a, int lda, const void* w, void* out, const int* offsets, const int* tiles,
                            const int* perm, int P, int E, int top, int N, int K, int mode, int act, float limit, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (N <= 0 || K <= 0 || K % 8 || lda % 8 || E <= 0 || top <= 0 || (((uintptr_t)a | (uintptr_t)w) & 15))
    return cima_fail(CIMA_E_SIZE, "moe_few: K %d and the row stride %d must be multiples of 8 and the operands 16-byte aligned", K, lda);
  if (mode != 0 && mode != 1) return cima_fail(CIMA_E_ARG, "moe_few: mode %d is neither 0 (gate | up) nor 1 (down)", mode);
  if (act < 0 || act >= CIMA_GATED_COUNT) return cima_fail(CIMA_E_ARG, "moe_few: activation code %d is unknown", act);
  const int per_block = 8 * (mode == 0 ? FEW_ROWS / 2 : FEW_ROWS);          // features of a block: its 8 warps' 
  const dim3 grid((unsigned)((P + BM - 1) / BM + E), (unsigned)((N + per_block - 1) / per_block));
  if (grid.y > 65535) return cima_fail(CIMA_E_SIZE, "moe_few: %d outputs exceed one launch", N);
  int rc;
  if (mode == 0) rc = cima_launch(k_moe_few<0>, grid, dim3(256), (size_t)0, stream, 1, (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)w, out, offsets, tiles, perm, E, top, N, K, act, limit);
  else rc = cima_launch(k_moe_few<1>, grid, dim3(256), (size_t)0, stream, 1, (const __nv_bfloat16*)a, lda, (const __nv_bfloat16*)w, out, offsets, tiles, perm, E, top, N, K, act, limit);
  return rc ? rc : cima_launch_result();
}
