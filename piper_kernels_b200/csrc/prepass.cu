// Quantisation prepass for the fused attention kernels (HBM-bound byte/float work).
//
// Restates, for sm_100a, what the reference project does before its tile loop:
//   * K (and V) sequence means, V channel abs-max        piper/reference.py:57-65, sage2pp/reference.py:25-28,49
//   * centred-row-range key order (stable ascending)      piper/reference.py:67-71
//   * INT8 Q / smoothed K in both scale granularities     attention/kernels/qk_quantization/int8/sage/reference.py:20-74
//   * Piper V: per-key INT8, stored transposed            piper/reference.py:27-37
//   * Sage V: per-channel E4M3, stored transposed         sage2pp/reference.py:25-28
// Arithmetic contract: scales are amax/range + 1e-7 with IEEE division, codes are
// clamp(rint(x / scale)), exactly as torch computes them on CPU.  Means are accumulated in
// FP64 and rounded once to FP32 (the summation order therefore does not matter).
//
// Every kernel reads each 16-bit input row with 16-byte vector loads when the pointers and
// strides allow it (ALIGNED), otherwise element by element.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <math.h>

#include <atomic>

#include "pk_internal.h"

namespace pk {
namespace {

constexpr int kThreads = 256;
constexpr int kBlockRows = 64;

struct TensorArg {
  const void* ptr;
  long long sb, sh, ss;  // element strides
};

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) {
  return __half2float(x);
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x);
}

// Loads 8 consecutive elements of a row as float.
template <typename T, bool ALIGNED>
__device__ __forceinline__ void load8(const T* p, float (&out)[8]) {
  if (ALIGNED) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = to_f32<T>(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = to_f32<T>(p[i]);
  }
}

__device__ __forceinline__ const void* head_ptr(const TensorArg& t, int bh, int heads, int elem_bytes) {
  const int b = bh / heads, h = bh % heads;
  return static_cast<const char*>(t.ptr) + (static_cast<long long>(b) * t.sb + static_cast<long long>(h) * t.sh) * elem_bytes;
}

// ---------------------------------------------------------------------------------------
// Column statistics: per (head, chunk of rows) FP64 column sums of K and V, or the column
// abs-max of V (Sage).  v_mode: 0 none, 1 sum, 2 abs-max.
// ---------------------------------------------------------------------------------------
template <typename T, int D, bool ALIGNED>
__global__ void __launch_bounds__(kThreads) colstat_partial_kernel(
    TensorArg k, TensorArg v, double* __restrict__ k_part, double* __restrict__ v_part, int sk, int heads,
    int chunks, int do_k, int v_mode) {
  constexpr int TPR = D / 8;           // threads per row
  constexpr int RPP = kThreads / TPR;  // rows per pass
  __shared__ double red[RPP * D];
  const int chunk = blockIdx.x, bh = blockIdx.y;
  const int cg = threadIdx.x % TPR, rl = threadIdx.x / TPR;
  const int r0 = chunk * kStatChunkRows;
  const int r1 = min(sk, r0 + kStatChunkRows);
  const T* kp = static_cast<const T*>(head_ptr(k, bh, heads, sizeof(T)));
  const T* vp = static_cast<const T*>(head_ptr(v, bh, heads, sizeof(T)));

  double ks[8], vs[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) ks[i] = 0.0, vs[i] = 0.0;
#pragma unroll 4
  for (int r = r0 + rl; r < r1; r += RPP) {
    float x[8];
    if (do_k) {
      load8<T, ALIGNED>(kp + static_cast<long long>(r) * k.ss + cg * 8, x);
#pragma unroll
      for (int i = 0; i < 8; ++i) ks[i] += static_cast<double>(x[i]);
    }
    if (v_mode) {
      load8<T, ALIGNED>(vp + static_cast<long long>(r) * v.ss + cg * 8, x);
      if (v_mode == 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) vs[i] += static_cast<double>(x[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) vs[i] = fmax(vs[i], static_cast<double>(fabsf(x[i])));
      }
    }
  }
  const long long out = (static_cast<long long>(bh) * chunks + chunk) * D;
  if (do_k) {
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rl * D + cg * 8 + i] = ks[i];
    __syncthreads();
    if (threadIdx.x < D) {
      double s = 0.0;
      for (int r = 0; r < RPP; ++r) s += red[r * D + threadIdx.x];
      k_part[out + threadIdx.x] = s;
    }
    __syncthreads();
  }
  if (v_mode) {
#pragma unroll
    for (int i = 0; i < 8; ++i) red[rl * D + cg * 8 + i] = vs[i];
    __syncthreads();
    if (threadIdx.x < D) {
      double s = 0.0;
      for (int r = 0; r < RPP; ++r) {
        const double x = red[r * D + threadIdx.x];
        s = (v_mode == 1) ? s + x : fmax(s, x);
      }
      v_part[out + threadIdx.x] = s;
    }
  }
}

// One thread per (head, feature): combine the chunk partials in chunk order.
__global__ void colstat_finalize_kernel(const double* __restrict__ k_part, const double* __restrict__ v_part,
                                        const float* __restrict__ k_override, const float* __restrict__ v_override,
                                        float* __restrict__ k_mean, float* __restrict__ v_out, int sk, int D,
                                        int chunks, int v_mode) {
  const int bh = blockIdx.x, d = threadIdx.x;
  if (d >= D) return;
  const long long base = static_cast<long long>(bh) * chunks * D + d;
  if (k_override) {
    k_mean[bh * D + d] = k_override[bh * D + d];
  } else {
    double s = 0.0;
    for (int c = 0; c < chunks; ++c) s += k_part[base + static_cast<long long>(c) * D];
    k_mean[bh * D + d] = static_cast<float>(s / static_cast<double>(sk));
  }
  if (v_mode == 0) {
    v_out[bh * D + d] = 0.f;
  } else if (v_mode == 1) {
    if (v_override) {
      v_out[bh * D + d] = v_override[bh * D + d];
    } else {
      double s = 0.0;
      for (int c = 0; c < chunks; ++c) s += v_part[base + static_cast<long long>(c) * D];
      v_out[bh * D + d] = static_cast<float>(s / static_cast<double>(sk));
    }
  } else {
    double m = 0.0;
    for (int c = 0; c < chunks; ++c) m = fmax(m, v_part[base + static_cast<long long>(c) * D]);
    // Sage V scale: amax / 2.25 + 1e-7 in FP32 (sage2pp/reference.py:26).
    v_out[bh * D + d] = __fadd_rn(__fdiv_rn(static_cast<float>(m), 2.25f), 1e-7f);
  }
}

// ---------------------------------------------------------------------------------------
// Centred row range r[n] = max_d |v[n,d] - mean[d]|, stored as the FP32 bit pattern (the
// values are non-negative, so unsigned integer order equals floating-point order).
// ---------------------------------------------------------------------------------------
constexpr int kRangePasses = 8;  // row passes per CTA of row_range_kernel

template <typename T, int D, bool ALIGNED>
__global__ void __launch_bounds__(kThreads) row_range_kernel(TensorArg v, const float* __restrict__ v_mean,
                                                             uint32_t* __restrict__ keys, int sk, int heads) {
  constexpr int TPR = D / 8;
  constexpr int RPP = kThreads / TPR;
  const int bh = blockIdx.y;
  const int cg = threadIdx.x % TPR, rl = threadIdx.x / TPR;
  const T* vp = static_cast<const T*>(head_ptr(v, bh, heads, sizeof(T)));
  float mean[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mean[i] = v_mean[bh * D + cg * 8 + i];
  float x[kRangePasses][8];
#pragma unroll
  for (int p = 0; p < kRangePasses; ++p) {  // all loads first: kRangePasses x 16 bytes in flight per thread
    const int r = (blockIdx.x * kRangePasses + p) * RPP + rl;
    if (r < sk) load8<T, ALIGNED>(vp + static_cast<long long>(r) * v.ss + cg * 8, x[p]);
  }
#pragma unroll
  for (int p = 0; p < kRangePasses; ++p) {
    const int r = (blockIdx.x * kRangePasses + p) * RPP + rl;
    float m = 0.f;
    if (r < sk) {
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(__fsub_rn(x[p][i], mean[i])));
    }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (r < sk && cg == 0) keys[static_cast<long long>(bh) * sk + r] = __float_as_uint(m);
  }
}

// ---------------------------------------------------------------------------------------
// Stable ascending sort of one head's keys: least-significant-digit radix sort, 8 bits per
// pass, one CTA per head.  Every warp owns a contiguous segment of the current order.  A pass
// is three steps with one CTA-wide barrier between them and none inside: (1) every warp counts
// the digits of its segment into its own histogram; (2) 256 threads turn the 32 x 256 counts
// into starting positions (digit-major, warp-minor, which keeps the order stable); (3) every
// warp walks its segment again, 32 keys at a time, ranks equal digits inside the group with
// match_any and moves keys and row indices to their positions.  A digit on which all keys agree
// (the sign and high exponent bits of a row range usually are) costs only step (1).  The row
// indices end in idx0 ("order").
// ---------------------------------------------------------------------------------------
constexpr int kSortThreads = 1024;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortBatch = 16;  // 32-key groups whose loads a warp issues before it ranks them

__global__ void __launch_bounds__(kSortThreads) segment_sort_kernel(uint32_t* __restrict__ keys0,
                                                                    uint32_t* __restrict__ keys1,
                                                                    int32_t* __restrict__ idx0,
                                                                    int32_t* __restrict__ idx1, int n) {
  __shared__ uint32_t cnt[kSortWarps][256];  // per-warp digit counts, then per-warp write positions
  __shared__ uint32_t total[256];
  __shared__ int skip[4];  // passes whose digit every key shares
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long seg = static_cast<long long>(blockIdx.x) * n;
  uint32_t* kbuf[2] = {keys0 + seg, keys1 + seg};
  int32_t* ibuf[2] = {idx0 + seg, idx1 + seg};
  // contiguous segment of this warp: a multiple of 32 keys so that groups never straddle warps
  const int per_warp = ((n + kSortWarps - 1) / kSortWarps + 31) / 32 * 32;
  const int w0 = min(n, warp * per_warp), w1 = min(n, w0 + per_warp);

  if (tid < 4) skip[tid] = 0;  // visible to all after the first barrier below
  int cur = 0;        // which buffer pair holds the current order
  bool first = true;  // the first pass that moves data reads the implicit identity permutation
  for (int pass = 0; pass < 4; ++pass) {
    const uint32_t* ksrc = kbuf[cur];
    const int shift = pass * 8;
    // (1) per-warp histograms
    for (int i = lane; i < 256; i += 32) cnt[warp][i] = 0;
    __syncwarp();
    for (int b0 = w0; b0 < w1; b0 += 32 * kSortBatch) {  // kSortBatch loads in flight per lane
      uint32_t kk[kSortBatch];
#pragma unroll
      for (int u = 0; u < kSortBatch; ++u) {
        const int i = b0 + u * 32 + lane;
        kk[u] = i < w1 ? ksrc[i] : 0u;
      }
#pragma unroll
      for (int u = 0; u < kSortBatch; ++u) {
        if (b0 + u * 32 + lane < w1) atomicAdd(&cnt[warp][(kk[u] >> shift) & 0xFF], 1u);
      }
    }
    __syncthreads();
    // (2) positions: thread d owns digit d
    if (tid < 256) {
      uint32_t sum = 0;
#pragma unroll 8
      for (int w = 0; w < kSortWarps; ++w) sum += cnt[w][tid];
      total[tid] = sum;
      if (sum == static_cast<uint32_t>(n)) skip[pass] = 1;
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan of the 256 digit totals, 8 per lane
      uint32_t c[8], sum = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        c[i] = total[lane * 8 + i];
        sum += c[i];
      }
      uint32_t incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      uint32_t run = incl - sum;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        total[lane * 8 + i] = run;
        run += c[i];
      }
    }
    __syncthreads();
    if (skip[pass]) continue;  // the same for every thread: written before the last barrier
    if (tid < 256) {
      uint32_t run = total[tid];
#pragma unroll 8
      for (int w = 0; w < kSortWarps; ++w) {
        const uint32_t c = cnt[w][tid];
        cnt[w][tid] = run;
        run += c;
      }
    }
    __syncthreads();
    // (3) stable scatter, warp by warp in segment order
    uint32_t* kdst = kbuf[cur ^ 1];
    const int32_t* isrc = ibuf[cur];
    int32_t* idst = ibuf[cur ^ 1];
    for (int b0 = w0; b0 < w1; b0 += 32 * kSortBatch) {
      uint32_t kk[kSortBatch];
      int32_t ii[kSortBatch];
#pragma unroll
      for (int u = 0; u < kSortBatch; ++u) {  // all loads of the batch first
        const int i = b0 + u * 32 + lane;
        kk[u] = 0;
        ii[u] = i;
        if (i < w1) {
          kk[u] = ksrc[i];
          if (!first) ii[u] = isrc[i];
        }
      }
#pragma unroll
      for (int u = 0; u < kSortBatch; ++u) {
        if (b0 + u * 32 >= w1) break;  // warp-uniform
        const bool valid = b0 + u * 32 + lane < w1;
        const uint32_t digit = valid ? ((kk[u] >> shift) & 0xFF) : 256u + lane;  // lanes past the end match nobody
        const uint32_t peers = __match_any_sync(0xffffffffu, digit);
        const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        const int leader = __ffs(peers) - 1;
        uint32_t base = 0;
        if (valid && rank == 0) {
          base = cnt[warp][digit];
          cnt[warp][digit] = base + __popc(peers);
        }
        base = __shfl_sync(0xffffffffu, base, leader);
        if (valid) {
          kdst[base + rank] = kk[u];
          idst[base + rank] = ii[u];
        }
        __syncwarp();
      }
    }
    __syncthreads();  // the next pass reads what every warp has just written (same CTA: visible after the barrier)
    cur ^= 1;
    first = false;
  }
  // the order is read from idx0
  if (first) {
    for (int i = tid; i < n; i += kSortThreads) ibuf[0][i] = i;
  } else if (cur == 1) {
    for (int i = tid; i < n; i += kSortThreads) ibuf[0][i] = ibuf[1][i];
  }
}

// ---------------------------------------------------------------------------------------
// INT8 quantisation of Q and of smoothed K.  One CTA per 64 rows; every thread keeps its
// share of the rows in registers between the abs-max and the rounding step, so the input is
// read exactly once.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ int round_clamp_i8(float x, float s) {
  const float q = rintf(__fdiv_rn(x, s));
  return static_cast<int>(fminf(fmaxf(q, -127.f), 127.f));
}

// Same result as round_clamp_i8(x, s) with r = fl(1 / s), without the IEEE division in the common
// case.  |x / s| < 128, so t = fl(x * r) is within 128 * (2^-24 + 2^-24) < 1.6e-5 of x / s, and the
// correctly rounded quotient within 7.7e-6 of it: when t is at least 1e-4 away from every
// half-integer, rint(t) equals rint(fl(x / s)); otherwise (about one element in 5000) the
// division is done.
__device__ __forceinline__ int round_clamp_i8_rcp(float x, float s, float r) {
  const float t = x * r;
  float q = rintf(t);
  if (fabsf(fabsf(t - q) - 0.5f) < 1e-4f) q = rintf(__fdiv_rn(x, s));
  return static_cast<int>(fminf(fmaxf(q, -127.f), 127.f));
}

template <typename T, int D, bool IS_KEY, bool ALIGNED>
__global__ void __launch_bounds__(kThreads) quantize_qk_kernel(
    TensorArg x, const float* __restrict__ mean, const int32_t* __restrict__ order, int8_t* __restrict__ codes,
    float* __restrict__ gscale, float* __restrict__ row_mul, int len, int len_pad, int heads, int per_thread,
    int groups_per_head, float mul) {
  constexpr int TPR = D / 8;
  constexpr int RPP = kThreads / TPR;
  constexpr int NP = kBlockRows / RPP;
  __shared__ float row_max[kBlockRows];
  __shared__ float row_scale[kBlockRows];
  const int bh = blockIdx.y, blk = blockIdx.x;
  const int cg = threadIdx.x % TPR, rl = threadIdx.x / TPR;
  const T* xp = static_cast<const T*>(head_ptr(x, bh, heads, sizeof(T)));

  float mu[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mu[i] = IS_KEY ? mean[bh * D + cg * 8 + i] : 0.f;

  // All row indices first, then all row loads, then the arithmetic: NP 16-byte loads per thread
  // are in flight at once (two dependent levels when rows are gathered through `order`).
  float vals[NP][8];
  long long src[NP];
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int r = blk * kBlockRows + p * RPP + rl;
    src[p] = -1;
    if (r < len) src[p] = (IS_KEY && order != nullptr) ? order[static_cast<long long>(bh) * len + r] : r;
  }
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    if (src[p] >= 0) {
      load8<T, ALIGNED>(xp + src[p] * x.ss + cg * 8, vals[p]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) vals[p][i] = 0.f;
    }
  }
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int lr = p * RPP + rl;
    float m = 0.f;
    if (src[p] >= 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (IS_KEY) vals[p][i] = __fsub_rn(vals[p][i], mu[i]);
        m = fmaxf(m, fabsf(vals[p][i]));
      }
    }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (cg == 0) row_max[lr] = m;
  }
  __syncthreads();
  if (threadIdx.x < kBlockRows) {  // two full warps: lane = row & 31
    const int r = threadIdx.x;
    const float own = row_max[r], other = row_max[r ^ 32];
    float g;
    if (!per_thread) {
      // one scale per 32 query rows (a warp) / per 64 key rows (both warps)
      g = IS_KEY ? fmaxf(own, other) : own;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) g = fmaxf(g, __shfl_xor_sync(0xffffffffu, g, o));
    } else if (!IS_KEY) {
      // rows {t, t+8, t+16, t+24} of each 32-row block (sage/reference.py:27-28)
      g = fmaxf(own, __shfl_xor_sync(0xffffffffu, own, 8));
      g = fmaxf(g, __shfl_xor_sync(0xffffffffu, g, 16));
    } else {
      // rows 8a + 2t + c, a < 8, c < 2 (sage/reference.py:46-47): every row that differs only in
      // bit 0 (c) or bits 3-5 (a)
      g = fmaxf(own, other);
      g = fmaxf(g, __shfl_xor_sync(0xffffffffu, g, 1));
      g = fmaxf(g, __shfl_xor_sync(0xffffffffu, g, 8));
      g = fmaxf(g, __shfl_xor_sync(0xffffffffu, g, 16));
    }
    const float s = __fadd_rn(__fdiv_rn(g, 127.f), 1e-7f);
    row_scale[r] = s;
    const int gr = blk * kBlockRows + r;
    if (gr < len_pad) row_mul[static_cast<long long>(bh) * len_pad + gr] = s * mul;
    if (per_thread) {
      if (gr < len) gscale[static_cast<long long>(bh) * groups_per_head + gr] = s;
    } else if (IS_KEY) {
      if (r == 0) gscale[static_cast<long long>(bh) * groups_per_head + blk] = s;
    } else if ((r & 31) == 0) {
      const int gi = blk * 2 + (r >> 5);
      if (gi < groups_per_head) gscale[static_cast<long long>(bh) * groups_per_head + gi] = s;
    }
  }
  __syncthreads();
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int lr = p * RPP + rl;
    const int r = blk * kBlockRows + lr;
    if (r >= len_pad) continue;
    const float s = row_scale[lr];
    const float rs = __fdiv_rn(1.f, s);
    uint32_t w[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t acc = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) acc |= (static_cast<uint32_t>(round_clamp_i8_rcp(vals[p][h * 4 + i], s, rs)) & 0xFFu) << (8 * i);
      w[h] = acc;
    }
    *reinterpret_cast<uint2*>(codes + (static_cast<long long>(bh) * len_pad + r) * D + cg * 8) = make_uint2(w[0], w[1]);
  }
}

// ---------------------------------------------------------------------------------------
// V quantisation.  Codes are written transposed, [head, feature, key], so that a 64-key tile
// is a K-major B operand of the PV product.  PIPER: per-key INT8 of (v - mean), plus
// log2(scale) and 1/scale per key.  SAGE: per-channel E4M3.
// ---------------------------------------------------------------------------------------
template <typename T, int D, bool SAGE, bool ALIGNED>
__global__ void __launch_bounds__(kThreads) quantize_v_kernel(
    TensorArg v, const float* __restrict__ v_mean_or_scale, const int32_t* __restrict__ order,
    uint8_t* __restrict__ codes_t, float* __restrict__ v_scale, float* __restrict__ col_add,
    float* __restrict__ col_inv, int sk, int sk_pad, int heads) {
  constexpr int TPR = D / 8;
  constexpr int RPP = kThreads / TPR;
  constexpr int NP = kBlockRows / RPP;  // adjacent keys per thread: 4 (head_dim 128) or 2 (64)
  constexpr int WPR = kBlockRows / 4;   // 32-bit words per feature row of the transposed tile
  static_assert(NP == 4 || NP == 2, "a thread's keys fill a word or half a word");
  // Transposed tile [feature][64 keys]; a thread owns NP adjacent keys, so it writes one (half) word
  // per feature.  The word position is rotated by the feature group so that the 16 (8) threads that
  // hold the same keys of different feature groups hit different banks.
  __shared__ __align__(16) uint32_t tile[D * WPR];
  const int bh = blockIdx.y, blk = blockIdx.x;
  const int cg = threadIdx.x % TPR, rl = threadIdx.x / TPR;
  const T* vp = static_cast<const T*>(head_ptr(v, bh, heads, sizeof(T)));

  float aux[8];  // PIPER: mean; SAGE: channel scale
#pragma unroll
  for (int i = 0; i < 8; ++i) aux[i] = v_mean_or_scale[bh * D + cg * 8 + i];

  uint32_t packed[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) packed[i] = 0;
  // row indices, then all row loads (NP 16-byte loads per thread in flight), then the arithmetic
  long long src[NP];
  float xs[NP][8];
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int r = blk * kBlockRows + rl * NP + p;
    src[p] = -1;
    if (r < sk) src[p] = (!SAGE && order != nullptr) ? order[static_cast<long long>(bh) * sk + r] : r;
  }
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    if (src[p] >= 0) {
      load8<T, ALIGNED>(vp + src[p] * v.ss + cg * 8, xs[p]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) xs[p][i] = 0.f;
    }
  }
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int lr = rl * NP + p;
    const int r = blk * kBlockRows + lr;
    float (&x)[8] = xs[p];
    float m = 0.f;
    if (r < sk && !SAGE) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[i] = __fsub_rn(x[i], aux[i]);
        m = fmaxf(m, fabsf(x[i]));
      }
    }
    if (!SAGE) {
#pragma unroll
      for (int o = TPR / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      const float s = __fadd_rn(__fdiv_rn(m, 127.f), 1e-7f);
      const float rs = __fdiv_rn(1.f, s);
      if (cg == 0) {
        const long long o = static_cast<long long>(bh) * sk_pad + r;
        if (r < sk) {
          v_scale[static_cast<long long>(bh) * sk + r] = s;
          col_add[o] = log2f(s);
          col_inv[o] = rs;
        } else {
          col_add[o] = -INFINITY;
          col_inv[o] = 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) packed[i] |= (static_cast<uint32_t>(round_clamp_i8_rcp(x[i], s, rs)) & 0xFFu) << (8 * p);
    } else {
      if (cg == 0) col_add[static_cast<long long>(bh) * sk_pad + r] = (r < sk) ? 0.f : -INFINITY;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float q = __fdiv_rn(x[i], aux[i]);
        packed[i] |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3)) << (8 * p);
      }
    }
  }
  {
    const int key0 = rl * NP;                   // first of this thread's keys within the tile
    const int word = ((key0 >> 2) + cg) % WPR;  // rotated word position
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t* row = tile + (cg * 8 + i) * WPR;
      if (NP == 4) row[word] = packed[i];
      else reinterpret_cast<uint16_t*>(row)[word * 2 + ((key0 >> 1) & 1)] = static_cast<uint16_t>(packed[i]);
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < D * WPR; idx += kThreads) {
    const int d = idx / WPR, w = idx % WPR;
    const uint32_t val = tile[d * WPR + (w + d / 8) % WPR];
    *reinterpret_cast<uint32_t*>(codes_t + (static_cast<long long>(bh) * D + d) * sk_pad + blk * kBlockRows + w * 4) = val;
  }
}

__global__ void zero_words_kernel(int32_t* p, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = 0;
}

bool aligned16(const void* ptr, const int64_t* s, int elem_bytes) {
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return false;
  for (int i = 0; i < 3; ++i)
    if ((s[i] * elem_bytes) & 15) return false;
  return true;
}

template <typename T, int D, bool ALIGNED>
int run_prepass(const pk_problem& p, const Layout& L, Algo algo, cudaStream_t st, int parts) {
  const TensorArg q{p.q, p.q_stride[0], p.q_stride[1], p.q_stride[2]};
  const TensorArg k{p.k, p.k_stride[0], p.k_stride[1], p.k_stride[2]};
  const TensorArg v{p.v, p.v_stride[0], p.v_stride[1], p.v_stride[2]};
  const int BH = L.BH;
  const bool sage = algo == kSage;
  const bool center = !sage && p.center_value;
  const bool sort = !sage && p.sort_value_rows;
  const int per_thread = p.qk_granularity == PK_QK_PER_THREAD;

  zero_words_kernel<<<1, 32, 0, st>>>(at<int32_t>(p, L.status), 16);
  const bool do_kv = (parts & kPrepassKV) != 0, do_q = (parts & kPrepassQ) != 0;

  if (do_q) {
    quantize_qk_kernel<T, D, false, ALIGNED><<<dim3(L.sq_pad / kBlockRows, BH), kThreads, 0, st>>>(
        q, nullptr, nullptr, at<int8_t>(p, L.q_codes), at<float>(p, L.q_gscale), at<float>(p, L.q_mul), L.Sq,
        L.sq_pad, p.heads, per_thread, L.q_groups, p.scale * kLog2e);
  }
  if (!do_kv) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PK_ERR_CUDA, "prepass launch failed: %s", cuda_err(e));
    return PK_OK;
  }

  // 1. column statistics
  const int do_k = p.k_mean_override == nullptr;
  const int v_mode = sage ? 2 : ((center && p.v_mean_override == nullptr) ? 1 : 0);
  if (do_k || v_mode) {
    colstat_partial_kernel<T, D, ALIGNED><<<dim3(L.chunks, BH), kThreads, 0, st>>>(
        k, v, at<double>(p, L.k_part), at<double>(p, L.v_part), L.Sk, p.heads, L.chunks, do_k, v_mode);
  }
  // v slot: piper -> mean [BH,D]; sage -> channel scale [BH,D] (stored in the v_scale view)
  float* v_stat = sage ? at<float>(p, L.v_scale) : at<float>(p, L.v_mean);
  const int fin_mode = sage ? 2 : (center ? 1 : 0);
  colstat_finalize_kernel<<<BH, D, 0, st>>>(at<double>(p, L.k_part), at<double>(p, L.v_part), p.k_mean_override,
                                            center ? p.v_mean_override : nullptr, at<float>(p, L.k_mean), v_stat,
                                            L.Sk, D, L.chunks, fin_mode);

  // 2. key order
  const int32_t* order = nullptr;
  if (sort) {
    constexpr int RPB = kRangePasses * (kThreads / (D / 8));  // rows per CTA
    row_range_kernel<T, D, ALIGNED><<<dim3((L.Sk + RPB - 1) / RPB, BH), kThreads, 0, st>>>(
        v, at<float>(p, L.v_mean), at<uint32_t>(p, L.range), L.Sk, p.heads);
    segment_sort_kernel<<<BH, kSortThreads, 0, st>>>(at<uint32_t>(p, L.range), at<uint32_t>(p, L.keys_alt),
                                                     at<int32_t>(p, L.idx_a), at<int32_t>(p, L.idx_b), L.Sk);
    order = at<int32_t>(p, L.idx_a);
  }

  // 3. K codes
  quantize_qk_kernel<T, D, true, ALIGNED><<<dim3(L.sk_pad / kBlockRows, BH), kThreads, 0, st>>>(
      k, at<float>(p, L.k_mean), order, at<int8_t>(p, L.k_codes), at<float>(p, L.k_gscale), at<float>(p, L.k_mul),
      L.Sk, L.sk_pad, p.heads, per_thread, L.k_groups, 1.0f);

  // 4. V codes
  if (sage) {
    quantize_v_kernel<T, D, true, ALIGNED><<<dim3(L.sk_pad / kBlockRows, BH), kThreads, 0, st>>>(
        v, at<float>(p, L.v_scale), nullptr, at<uint8_t>(p, L.v_codes), nullptr, at<float>(p, L.k_add), nullptr,
        L.Sk, L.sk_pad, p.heads);
  } else {
    quantize_v_kernel<T, D, false, ALIGNED><<<dim3(L.sk_pad / kBlockRows, BH), kThreads, 0, st>>>(
        v, at<float>(p, L.v_mean), order, at<uint8_t>(p, L.v_codes), at<float>(p, L.v_scale), at<float>(p, L.k_add),
        at<float>(p, L.k_inv), L.Sk, L.sk_pad, p.heads);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PK_ERR_CUDA, "prepass launch failed: %s", cuda_err(e));
  return PK_OK;
}

template <typename T, int D>
int run_prepass_a(const pk_problem& p, const Layout& L, Algo algo, cudaStream_t st, int parts) {
  const int eb = 2;
  // only the tensors this call reads decide between vector and element-wise loads
  const bool al = (!(parts & kPrepassQ) || aligned16(p.q, p.q_stride, eb)) &&
                  (!(parts & kPrepassKV) || (aligned16(p.k, p.k_stride, eb) && aligned16(p.v, p.v_stride, eb)));
  return al ? run_prepass<T, D, true>(p, L, algo, st, parts) : run_prepass<T, D, false>(p, L, algo, st, parts);
}

}  // namespace

int launch_prepass(const pk_problem& p, const Layout& L, Algo algo, cudaStream_t st, int parts) {
  if (p.in_dtype == PK_F16) {
    return p.head_dim == 128 ? run_prepass_a<__half, 128>(p, L, algo, st, parts) : run_prepass_a<__half, 64>(p, L, algo, st, parts);
  }
  return p.head_dim == 128 ? run_prepass_a<__nv_bfloat16, 128>(p, L, algo, st, parts)
                           : run_prepass_a<__nv_bfloat16, 64>(p, L, algo, st, parts);
}

// ---------------------------------------------------------------------------------------
// K / V sequence means without any caller-provided scratch.
//
// Some hosts that embed this library may not allocate device memory at the point where they
// need the means: code running under a memory pool that has been frozen for the lifetime of a
// serving process, plug-ins that are handed fixed input/output buffers by their runtime, or
// callers that must not disturb an allocator whose state is being recorded.  For them the
// per-chunk FP64 partial sums live in a fixed array inside the library image instead of in a
// workspace.  Every device that loads the library carries the array (8 MiB) until exit.
// ---------------------------------------------------------------------------------------
namespace {

constexpr long long kStaticPartialsPerTensor = 512 * 1024;  // FP64 words: batch*heads*ceil(kv_len/512)*head_dim
static __device__ __align__(256) double g_static_mean_partials[2 * kStaticPartialsPerTensor];

// Device address of the array, looked up once per device while that device is current.  The
// array's name in host code is only a handle for this lookup, never a pointer to pass along.
double* static_partials_for_current_device(int device, cudaError_t* err) {
  // Threads that make the first call on a device at the same time all look the address up and
  // store the same value; later calls read it without touching the runtime.
  static std::atomic<double*> cache[64];
  *err = cudaSuccess;
  if (device >= 0 && device < 64) {
    double* known = cache[device].load(std::memory_order_acquire);
    if (known != nullptr) return known;
  }
  double* ptr = nullptr;
  *err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_mean_partials);
  if (*err != cudaSuccess) return nullptr;
  if (device >= 0 && device < 64) cache[device].store(ptr, std::memory_order_release);
  return ptr;
}

template <typename T, int D>
void launch_means_static(const pk_problem& p, double* scratch, float* k_mean, float* v_mean, int chunks,
                         cudaStream_t st) {
  const TensorArg k{p.k, p.k_stride[0], p.k_stride[1], p.k_stride[2]};
  const TensorArg v{p.v, p.v_stride[0], p.v_stride[1], p.v_stride[2]};
  const int BH = p.batch * p.heads;
  double* k_part = scratch;
  double* v_part = scratch + kStaticPartialsPerTensor;
  const bool al = aligned16(p.k, p.k_stride, 2) && aligned16(p.v, p.v_stride, 2);
  // Each launch overwrites every partial it later reads, so nothing needs clearing first.
  if (al) colstat_partial_kernel<T, D, true><<<dim3(chunks, BH), kThreads, 0, st>>>(k, v, k_part, v_part, p.kv_len, p.heads, chunks, 1, 1);
  else colstat_partial_kernel<T, D, false><<<dim3(chunks, BH), kThreads, 0, st>>>(k, v, k_part, v_part, p.kv_len, p.heads, chunks, 1, 1);
  colstat_finalize_kernel<<<BH, D, 0, st>>>(k_part, v_part, nullptr, nullptr, k_mean, v_mean, p.kv_len, D, chunks, 1);
}

}  // namespace

int kv_means_static(const pk_problem& p, float* k_mean, float* v_mean) {
  const int chunks = (p.kv_len + kStatChunkRows - 1) / kStatChunkRows;
  const long long need = static_cast<long long>(p.batch) * p.heads * chunks * p.head_dim;
  if (need > kStaticPartialsPerTensor)
    return fail(PK_ERR_BAD_ARG,
                "pk_kv_means_static: batch*heads*ceil(kv_len/512)*head_dim = %lld exceeds the built-in scratch of %lld "
                "partial sums; use pk_piper_prepare with a workspace instead",
                need, kStaticPartialsPerTensor);
  cudaError_t e;
  double* scratch = static_partials_for_current_device(p.device, &e);
  if (!scratch) return fail(PK_ERR_CUDA, "pk_kv_means_static: cudaGetSymbolAddress failed: %s", cuda_err(e));
  cudaStream_t st = static_cast<cudaStream_t>(p.stream);
  if (p.in_dtype == PK_F16) {
    if (p.head_dim == 128) launch_means_static<__half, 128>(p, scratch, k_mean, v_mean, chunks, st);
    else launch_means_static<__half, 64>(p, scratch, k_mean, v_mean, chunks, st);
  } else {
    if (p.head_dim == 128) launch_means_static<__nv_bfloat16, 128>(p, scratch, k_mean, v_mean, chunks, st);
    else launch_means_static<__nv_bfloat16, 64>(p, scratch, k_mean, v_mean, chunks, st);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PK_ERR_CUDA, "pk_kv_means_static launch failed: %s", cuda_err(e));
  return PK_OK;
}

}  // namespace pk
