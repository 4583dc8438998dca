// Rotary position encoding of q and k, and the append of k and v to the paged cache, in one pass
// over a step's rows.
//
// qkv is [T, ld]: q heads, then k heads, then v heads of each row.  q and k are rotated in place
// (prefill attention reads them from this buffer); the rotated k and the v are also written to the
// position's place in the layer's pages.  The angle p * inv_freq[i] and its sine and cosine are
// float32 (sincosf, not the fast approximations); inv_freq[i] = theta^(-2i / rotary_dim) comes from
// the host, computed in float64.  Pair (i, i + rotary_dim/2) of a head rotates:
//   u_i' = u_i cos a - u_j sin a,   u_j' = u_i sin a + u_j cos a        (src/kernels.cu:397-414)
// Sine and cosine are multiplied by `amp` (1 for a plain rotation; a rescaled table may ask for another amplitude).
// Dimensions from rotary_dim on pass through.  Append: src/kernels.cu:440-454 (one sequence,
// [kv_heads, max_seq, dim]); here the place comes from the slot's block table.
#include "common.cuh"

template <typename TA>
__global__ void __launch_bounds__(256)
k_rope_append(TA* __restrict__ qkv, int ld, const float* __restrict__ inv_freq, int rotary_dim,
              const int* __restrict__ row_pos, const int* __restrict__ row_seq, const int* __restrict__ seq_slot,
              const int* __restrict__ seq_len, TA* __restrict__ cache_in, CimaPaged pg, int nh, int nkv, int hd, float amp) {
  cima_pdl_wait();
  __shared__ float cs[128], sn[128];
  const int row = blockIdx.x;
  const int pos = row_pos[row];
  const int half = rotary_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    cs[i] = c * amp;
    sn[i] = s * amp;
  }
  __syncthreads();
  TA* base = qkv + (size_t)row * ld;
  // In a ring of pages a long prompt wraps: a position whose place a later position of the same
  // step takes is not written at all (two rows of one launch must not write one place).
  TA* cache = cache_in;
  if (cache && pg.ring && pos + pg.ring * pg.page_size < seq_len[row_seq[row]]) cache = nullptr;
  const int slot = cache ? seq_slot[row_seq[row]] : 0;
  // rotation pairs of q heads [0, nh) and k heads [nh, nh + nkv)
  const int npairs = (nh + nkv) * half;
  for (int idx = threadIdx.x; idx < npairs; idx += blockDim.x) {
    const int head = idx / half, i = idx - head * half;
    TA* u = base + (size_t)head * hd;
    const float a = cima_to_f32<TA>(u[i]), b = cima_to_f32<TA>(u[i + half]);
    const TA ra = cima_from_f32<TA>(a * cs[i] - b * sn[i]);
    const TA rb = cima_from_f32<TA>(a * sn[i] + b * cs[i]);
    u[i] = ra;
    u[i + half] = rb;
    if (cache && head >= nh) {
      TA* dst = cache + pg.offset(slot, pos, 0, head - nh);
      dst[i] = ra;
      dst[i + half] = rb;
    }
  }
  if (!cache) return;
  // k dimensions that do not rotate
  const int rest = hd - rotary_dim;
  for (int idx = threadIdx.x; idx < nkv * rest; idx += blockDim.x) {
    const int head = idx / rest, d = rotary_dim + (idx - head * rest);
    cache[pg.offset(slot, pos, 0, head) + d] = base[(size_t)(nh + head) * hd + d];
  }
  // v
  for (int idx = threadIdx.x; idx < nkv * hd; idx += blockDim.x) {
    const int head = idx / hd, d = idx - head * hd;
    cache[pg.offset(slot, pos, 1, head) + d] = base[(size_t)(nh + nkv + head) * hd + d];
  }
}

// The same for bfloat16 rows whose halves are multiples of 8: a thread takes 8 consecutive pairs, i.e. two
// 16-byte pieces of a head, and every access to the row and to the cache is 16 bytes wide.  Same arithmetic,
// element by element, as the kernel above.
__global__ void __launch_bounds__(256)
k_rope_append_bf16x8(__nv_bfloat16* __restrict__ qkv, int ld, const float* __restrict__ inv_freq, int rotary_dim,
                     const int* __restrict__ row_pos, const int* __restrict__ row_seq, const int* __restrict__ seq_slot,
                     const int* __restrict__ seq_len, __nv_bfloat16* __restrict__ cache_in, CimaPaged pg, int nh, int nkv,
                     int hd, float amp) {
  cima_pdl_wait();
  __shared__ float cs[128], sn[128];
  const int row = blockIdx.x;
  const int pos = row_pos[row];
  const int half = rotary_dim >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf((float)pos * inv_freq[i], &s, &c);
    cs[i] = c * amp;
    sn[i] = s * amp;
  }
  __syncthreads();
  __nv_bfloat16* base = qkv + (size_t)row * ld;
  __nv_bfloat16* cache = cache_in;
  if (cache && pg.ring && pos + pg.ring * pg.page_size < seq_len[row_seq[row]]) cache = nullptr;
  const int slot = cache ? seq_slot[row_seq[row]] : 0;
  const int h8 = half >> 3;                              // groups of 8 pairs per head
  for (int idx = threadIdx.x; idx < (nh + nkv) * h8; idx += blockDim.x) {
    const int head = idx / h8, i = (idx - head * h8) * 8;
    __nv_bfloat16* u = base + (size_t)head * hd;
    uint4 av = *reinterpret_cast<const uint4*>(u + i), bv = *reinterpret_cast<const uint4*>(u + i + half);
    __nv_bfloat16* a = reinterpret_cast<__nv_bfloat16*>(&av);
    __nv_bfloat16* b = reinterpret_cast<__nv_bfloat16*>(&bv);
#pragma unroll
    for (int e = 0; e < 8; e++) {
      const float x = __bfloat162float(a[e]), y = __bfloat162float(b[e]);
      a[e] = __float2bfloat16_rn(x * cs[i + e] - y * sn[i + e]);
      b[e] = __float2bfloat16_rn(x * sn[i + e] + y * cs[i + e]);
    }
    *reinterpret_cast<uint4*>(u + i) = av;
    *reinterpret_cast<uint4*>(u + i + half) = bv;
    if (cache && head >= nh) {
      __nv_bfloat16* dst = cache + pg.offset(slot, pos, 0, head - nh);
      *reinterpret_cast<uint4*>(dst + i) = av;
      *reinterpret_cast<uint4*>(dst + i + half) = bv;
    }
  }
  if (!cache) return;
  const int rest8 = (hd - rotary_dim) >> 3;              // k dimensions that do not rotate
  for (int idx = threadIdx.x; idx < nkv * rest8; idx += blockDim.x) {
    const int head = idx / rest8, d = rotary_dim + (idx - head * rest8) * 8;
    *reinterpret_cast<uint4*>(cache + pg.offset(slot, pos, 0, head) + d) =
        *reinterpret_cast<const uint4*>(base + (size_t)(nh + head) * hd + d);
  }
  const int hd8 = hd >> 3;
  for (int idx = threadIdx.x; idx < nkv * hd8; idx += blockDim.x) {
    const int head = idx / hd8, d = (idx - head * hd8) * 8;
    *reinterpret_cast<uint4*>(cache + pg.offset(slot, pos, 1, head) + d) =
        *reinterpret_cast<const uint4*>(base + (size_t)(nh + nkv + head) * hd + d);
  }
}


// The general form: a warp a head of a row.  Before the rotation the first `norm_dim` values of every q and k head are
// divided by their root mean square (eps inside the root) and multiplied by a weight of `norm_dim` values, one for all
// q heads and one for all k heads (no norm where the weights are null); and a row holds `nv` value heads behind its key
// heads (nv <= nkv: neighbouring key heads share a value head), which go to the first nv heads of the pages' value
// plane.  Sums of squares, the norm, the angle and the rotation are float32; one rounding at the store.
// VEC 4: a lane takes four neighbouring values at a time (one 8- or 16-byte load and store); the launch chooses it where
// head size and row stride are multiples of 4 and the pointers are aligned, else VEC 1.
template <typename TA> __device__ __forceinline__ void rope_load4(const TA* p, float* f);
template <> __device__ __forceinline__ void rope_load4<float>(const float* p, float* f) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  f[0] = t.x; f[1] = t.y; f[2] = t.z; f[3] = t.w;
}
template <> __device__ __forceinline__ void rope_load4<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <typename TA> struct RopePack4;
template <> struct RopePack4<float> {
  float4 t;
  __device__ __forceinline__ RopePack4(const float* f) : t(make_float4(f[0], f[1], f[2], f[3])) {}
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = t; }
};
template <> struct RopePack4<__nv_bfloat16> {
  uint2 t;
  __device__ __forceinline__ RopePack4(const float* f) {
    *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(f[0], f[1]);
    *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(f[2], f[3]);
  }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint2*>(p) = t; }
};

template <typename TA, int VEC>
__global__ void __launch_bounds__(128)
k_norm_rope_append(TA* __restrict__ qkv, int ld, const float* __restrict__ inv_freq, int rotary_dim,
                   const int* __restrict__ row_pos, const int* __restrict__ row_seq, const int* __restrict__ seq_slot,
                   const int* __restrict__ seq_len, TA* __restrict__ cache_in, CimaPaged pg, int nh, int nkv, int nv, int hd,
                   const float* __restrict__ q_norm, const float* __restrict__ k_norm, int norm_dim, float eps, float amp) {
  cima_pdl_wait();
  __shared__ __align__(16) float vals[4][256];
  __shared__ float rot_cos[128], rot_sin[128];
  const int row = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.x * 4 + warp;
  const int pos = row_pos[row];
  const int half = rotary_dim >> 1;
  if (blockIdx.x * 4 < nh + nkv) {                     // the row's angles once for the block's heads
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      float sv, cv;
      sincosf((float)pos * inv_freq[i], &sv, &cv);
      rot_sin[i] = sv * amp;
      rot_cos[i] = cv * amp;
    }
    __syncthreads();
  }
  if (head >= nh + nkv + nv) return;
  TA* cache = cache_in;
  if (cache && pg.ring && pos + pg.ring * pg.page_size < seq_len[row_seq[row]]) cache = nullptr;
  const int slot = cache ? seq_slot[row_seq[row]] : 0;
  TA* u = qkv + (size_t)row * ld + (size_t)head * hd;
  if (head >= nh + nkv) {                              // a value head: to the pages as it is
    if (!cache) return;
    TA* dst = cache + pg.offset(slot, pos, 1, head - nh - nkv);
    if (VEC == 4) {
      for (int d = lane * 4; d < hd; d += 128) {
        if (sizeof(TA) == 2) *reinterpret_cast<uint2*>(dst + d) = *reinterpret_cast<const uint2*>(u + d);
        else *reinterpret_cast<float4*>(dst + d) = *reinterpret_cast<const float4*>(u + d);
      }
    } else {
      for (int d = lane; d < hd; d += 32) dst[d] = u[d];
    }
    return;
  }
  const float* w = head < nh ? q_norm : k_norm;
  float* x = vals[warp];
  float ss = 0.f;
  if (VEC == 4) {
    for (int d = lane * 4; d < hd; d += 128) {
      float f[4];
      rope_load4<TA>(u + d, f);
      *reinterpret_cast<float4*>(x + d) = make_float4(f[0], f[1], f[2], f[3]);
#pragma unroll
      for (int e = 0; e < 4; e++)
        if (d + e < norm_dim) ss = fmaf(f[e], f[e], ss);
    }
  } else {
    for (int d = lane; d < hd; d += 32) {
      const float v = cima_to_f32<TA>(u[d]);
      x[d] = v;
      if (d < norm_dim) ss = fmaf(v, v, ss);
    }
  }
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (VEC == 4) __syncwarp();                          // the norm's loop reads what other lanes wrote
  if (w) {
    const float r = 1.0f / sqrtf(ss / (float)norm_dim + eps);
    for (int d = lane; d < norm_dim; d += 32) x[d] = x[d] * r * w[d];
  }
  __syncwarp();
  TA* dst = (cache && head >= nh) ? cache + pg.offset(slot, pos, 0, head - nh) : nullptr;
  auto turned = [&](int d) {
    float y = x[d];
    if (d < rotary_dim) {
      const int i = d < half ? d : d - half;
      const float sn = rot_sin[i], cs = rot_cos[i];
      y = d < half ? x[d] * cs - x[d + half] * sn : x[d - half] * sn + x[d] * cs;
    }
    return y;
  };
  if (VEC == 4) {
    for (int d = lane * 4; d < hd; d += 128) {
      const float f[4] = {turned(d), turned(d + 1), turned(d + 2), turned(d + 3)};
      const RopePack4<TA> r(f);
      r.store(u + d);
      if (dst) r.store(dst + d);
    }
  } else {
    for (int d = lane; d < hd; d += 32) {
      const TA r = cima_from_f32<TA>(turned(d));
      u[d] = r;
      if (dst) dst[d] = r;
    }
  }
}

// cache may be null (a layer that reads another layer's keys and values writes none).
// nv: value heads of a row (nkv unless key heads share value heads); q_norm / k_norm (both or neither): the weights of
// a norm over the first norm_dim values of every q / k head before the rotation.
// seq_len[i] is the length of sequence i after this step.
extern "C" int cima_rope_append(void* qkv, int dtype, int ld, const float* inv_freq, int rotary_dim,
                                const int* row_pos, const int* row_seq, const int* seq_slot, const int* seq_len,
                                void* cache, const int* table, int table_width, int ring, int page_size,
                                int T, int nh, int nkv, int hd, int nv, const float* q_norm, const float* k_norm, int norm_dim,
                                float eps, float amp, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || hd > 256 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1))
    return cima_fail(CIMA_E_SIZE, "rope_append: head_dim %d (at most 256) and an even rotary_dim %d <= head_dim are needed", hd, rotary_dim);
  if (nv < 0 || nv > nkv || (nv > 0 && nkv % nv)) return cima_fail(CIMA_E_SIZE, "rope_append: %d value heads must divide the %d key heads", nv, nkv);
  if (ld < (nh + nkv + nv) * hd) return cima_fail(CIMA_E_SIZE, "rope_append: row stride %d is smaller than (heads + key heads + value heads) * head_dim = %d", ld, (nh + nkv + nv) * hd);
  if ((q_norm != nullptr) != (k_norm != nullptr) || (q_norm && (norm_dim <= 0 || norm_dim > hd)))
    return cima_fail(CIMA_E_ARG, "rope_append: the norm takes weights for q and for k and 1 <= norm_dim %d <= head_dim %d", norm_dim, hd);
  if (cache && (page_size <= 0 || table_width <= 0)) return cima_fail(CIMA_E_SIZE, "rope_append: page size %d and table width %d must be positive", page_size, table_width);
  CimaPaged pg{table, table_width, ring, page_size, nkv, hd};
  if (q_norm || nv != nkv) {
    const dim3 grid((unsigned)((nh + nkv + nv + 3) / 4), (unsigned)T);
    if (T > 65535) return cima_fail(CIMA_E_SIZE, "rope_append: %d rows exceed one launch of the general kernel; the caller cuts them", T);
    int rc_;
    const size_t bytes = dtype == CIMA_F32 ? 4 : 2;
    const bool vec = hd % 4 == 0 && ld % 4 == 0 && ((uintptr_t)qkv % (4 * bytes)) == 0 && ((uintptr_t)cache % (4 * bytes)) == 0;
    if (vec) {
      if (dtype == CIMA_F32) rc_ = cima_launch(k_norm_rope_append<float, 4>, grid, dim3(128), (size_t)0, stream, 1, (float*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (float*)cache, pg, nh, nkv, nv, hd, q_norm, k_norm, norm_dim, eps, amp);
      else if (dtype == CIMA_BF16) rc_ = cima_launch(k_norm_rope_append<__nv_bfloat16, 4>, grid, dim3(128), (size_t)0, stream, 1, (__nv_bfloat16*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (__nv_bfloat16*)cache, pg, nh, nkv, nv, hd, q_norm, k_norm, norm_dim, eps, amp);
      else return cima_fail(CIMA_E_DTYPE, "rope_append: dtype code %d is neither float32 nor bfloat16", dtype);
      return rc_ ? rc_ : cima_launch_result();
    }
    if (dtype == CIMA_F32) rc_ = cima_launch(k_norm_rope_append<float, 1>, grid, dim3(128), (size_t)0, stream, 1, (float*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (float*)cache, pg, nh, nkv, nv, hd, q_norm, k_norm, norm_dim, eps, amp);
    else if (dtype == CIMA_BF16) rc_ = cima_launch(k_norm_rope_append<__nv_bfloat16, 1>, grid, dim3(128), (size_t)0, stream, 1, (__nv_bfloat16*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (__nv_bfloat16*)cache, pg, nh, nkv, nv, hd, q_norm, k_norm, norm_dim, eps, amp);
    else return cima_fail(CIMA_E_DTYPE, "rope_append: dtype code %d is neither float32 nor bfloat16", dtype);
    return rc_ ? rc_ : cima_launch_result();
  }
  if (dtype == CIMA_F32)
    { int rc_ = cima_launch(k_rope_append<float>, dim3(T), dim3(256), (size_t)(0), stream, 1, (float*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (float*)cache, pg, nh, nkv, hd, amp); if (rc_) return rc_; }
  else if (dtype == CIMA_BF16 && rotary_dim % 16 == 0 && hd % 8 == 0 && ld % 8 == 0 && rotary_dim <= 256 &&
           (((uintptr_t)qkv | (uintptr_t)cache) & 15) == 0)
    { int rc_ = cima_launch(k_rope_append_bf16x8, dim3(T), dim3(256), (size_t)(0), stream, 1, (__nv_bfloat16*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (__nv_bfloat16*)cache, pg, nh, nkv, hd, amp); if (rc_) return rc_; }
  else if (dtype == CIMA_BF16)
    { int rc_ = cima_launch(k_rope_append<__nv_bfloat16>, dim3(T), dim3(256), (size_t)(0), stream, 1, (__nv_bfloat16*)qkv, ld, inv_freq, rotary_dim, row_pos, row_seq, seq_slot, seq_len, (__nv_bfloat16*)cache, pg, nh, nkv, hd, amp); if (rc_) return rc_; }
  else return cima_fail(CIMA_E_DTYPE, "rope_append: dtype code %d is neither float32 nor bfloat16", dtype);
  return cima_launch_result();
}
