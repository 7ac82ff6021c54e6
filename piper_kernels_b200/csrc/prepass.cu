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
constexpr int kQuantBlocks = 2;  // 64-row blocks per CTA of the quantize kernels (loads of all of them in flight)
constexpr int kStatBatch = 4;  // row passes of colstat_partial_kernel whose loads are issued together

constexpr int ceil_div(int a, int b) { return (a + b - 1) / b; }

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

// Eight consecutive elements of a row as loaded (16 bytes: four registers), converted on use.
template <typename T>
struct Raw8 {
  union {
    uint4 u;
    T e[8];
  };
  __device__ __forceinline__ Raw8() {}
};
template <typename T, bool ALIGNED>
__device__ __forceinline__ void load8raw(const T* p, Raw8<T>& out) {
  if (ALIGNED) {
    out.u = __ldg(reinterpret_cast<const uint4*>(p));
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) out.e[i] = p[i];
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
  cudaGridDependencySynchronize();  // launched chained: wait for the predecessor's writes
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
  // kStatBatch row passes at a time: all their loads are issued before the first sum (2 x
  // kStatBatch 16-byte loads in flight per thread); the rows are summed in row order.
  for (int rb = r0 + rl; rb < r1; rb += RPP * kStatBatch) {
    Raw8<T> kr[kStatBatch], vr[kStatBatch];
#pragma unroll
    for (int u = 0; u < kStatBatch; ++u) {
      const int r = rb + u * RPP;
      if (r < r1) {
        if (do_k) load8raw<T, ALIGNED>(kp + static_cast<long long>(r) * k.ss + cg * 8, kr[u]);
        if (v_mode) load8raw<T, ALIGNED>(vp + static_cast<long long>(r) * v.ss + cg * 8, vr[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kStatBatch; ++u) {
      const int r = rb + u * RPP;
      if (r < r1) {
        if (do_k) {
#pragma unroll
          for (int i = 0; i < 8; ++i) ks[i] += static_cast<double>(to_f32<T>(kr[u].e[i]));
        }
        if (v_mode == 1) {
#pragma unroll
          for (int i = 0; i < 8; ++i) vs[i] += static_cast<double>(to_f32<T>(vr[u].e[i]));
        } else if (v_mode == 2) {
#pragma unroll
          for (int i = 0; i < 8; ++i) vs[i] = fmax(vs[i], static_cast<double>(fabsf(to_f32<T>(vr[u].e[i]))));
        }
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

// One thread per (head, tensor, feature): combine the chunk partials in chunk order.
// Launched with 2 * D threads: the first D finish K, the others V.
__device__ __forceinline__ double combine_chunks(const double* __restrict__ part, long long base, int D, int chunks,
                                                 bool take_max) {
  constexpr int kBatch = 16;  // partials loaded together; they are combined in chunk order
  double s = 0.0;
  for (int c0 = 0; c0 < chunks; c0 += kBatch) {
    double x[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) x[u] = (c0 + u < chunks) ? part[base + static_cast<long long>(c0 + u) * D] : 0.0;
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (c0 + u < chunks) s = take_max ? fmax(s, x[u]) : s + x[u];
    }
  }
  return s;
}

__global__ void colstat_finalize_kernel(const double* __restrict__ k_part, const double* __restrict__ v_part,
                                        const float* __restrict__ k_override, const float* __restrict__ v_override,
                                        float* __restrict__ k_mean, float* __restrict__ v_out, int sk, int D,
                                        int chunks, int v_mode) {
  cudaGridDependencySynchronize();  // launched chained: wait for the predecessor's writes
  const int bh = blockIdx.x, d = threadIdx.x % D;
  const bool v_role = static_cast<int>(threadIdx.x) >= D;
  const long long base = static_cast<long long>(bh) * chunks * D + d;
  if (!v_role) {
    if (k_override) {
      k_mean[bh * D + d] = k_override[bh * D + d];
    } else {
      const double s = combine_chunks(k_part, base, D, chunks, false);
      k_mean[bh * D + d] = static_cast<float>(s / static_cast<double>(sk));
    }
  } else if (v_mode == 0) {
    v_out[bh * D + d] = 0.f;
  } else if (v_mode == 1) {
    if (v_override) {
      v_out[bh * D + d] = v_override[bh * D + d];
    } else {
      const double s = combine_chunks(v_part, base, D, chunks, false);
      v_out[bh * D + d] = static_cast<float>(s / static_cast<double>(sk));
    }
  } else {
    const double m = combine_chunks(v_part, base, D, chunks, true);
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
  cudaGridDependencySynchronize();  // launched chained: wait for the predecessor's writes
  constexpr int TPR = D / 8;
  constexpr int RPP = kThreads / TPR;
  const int bh = blockIdx.y;
  const int cg = threadIdx.x % TPR, rl = threadIdx.x / TPR;
  const T* vp = static_cast<const T*>(head_ptr(v, bh, heads, sizeof(T)));
  float mean[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) mean[i] = v_mean[bh * D + cg * 8 + i];
  Raw8<T> x[kRangePasses];
#pragma unroll
  for (int p = 0; p < kRangePasses; ++p) {  // all loads first: kRangePasses x 16 bytes in flight per thread
    const int r = (blockIdx.x * kRangePasses + p) * RPP + rl;
    if (r < sk) load8raw<T, ALIGNED>(vp + static_cast<long long>(r) * v.ss + cg * 8, x[p]);
  }
#pragma unroll
  for (int p = 0; p < kRangePasses; ++p) {
    const int r = (blockIdx.x * kRangePasses + p) * RPP + rl;
    float m = 0.f;
    if (r < sk) {
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(__fsub_rn(to_f32<T>(x[p].e[i]), mean[i])));
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

__device__ __forceinline__ void segment_sort_body(uint32_t* __restrict__ keys0, uint32_t* __restrict__ keys1,
                                                  int32_t* __restrict__ idx0, int32_t* __restrict__ idx1, int n,
                                                  int head) {
  __shared__ uint32_t cnt[kSortWarps][256];  // per-warp digit counts, then per-warp write positions
  __shared__ uint32_t total[256];
  __shared__ int skip[4];  // passes whose digit every key shares
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long seg = static_cast<long long>(head) * n;
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

__global__ void __launch_bounds__(kSortThreads) segment_sort_kernel(uint32_t* __restrict__ keys0,
                                                                    uint32_t* __restrict__ keys1,
                                                                    int32_t* __restrict__ idx0,
                                                                    int32_t* __restrict__ idx1, int n) {
  cudaGridDependencySynchronize();  // launched chained: wait for the predecessor's writes
  segment_sort_body(keys0, keys1, idx0, idx1, n, blockIdx.x);
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

// Eight loaded elements as four FP32 pairs.  BF16 is the high half of an FP32 word: a shift and a mask.
template <typename T>
__device__ __forceinline__ void unpack8(const Raw8<T>& raw, float2 (&f)[4]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const Raw8<__nv_bfloat16>& raw, float2 (&f)[4]) {
  const uint32_t w[4] = {raw.u.x, raw.u.y, raw.u.z, raw.u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ void unpack8<__half>(const Raw8<__half>& raw, float2 (&f)[4]) {
  const uint32_t w[4] = {raw.u.x, raw.u.y, raw.u.z, raw.u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) f[i] = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
}

// Maximum of a non-negative value over the aligned group of N lanes the caller belongs to
// (unsigned order of the bit patterns equals the order of non-negative floats): one warp
// reduction instead of log2(N) shuffle steps.  Every lane of the warp must call it.
template <int N>
__device__ __forceinline__ float group_max(float m) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t mask = (N == 32 ? 0xffffffffu : ((1u << N) - 1u)) << (lane & ~static_cast<uint32_t>(N - 1));
  return __uint_as_float(__reduce_max_sync(mask, __float_as_uint(m)));
}

__device__ __forceinline__ float absmax3(float m, float a, float b) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(m), "f"(fabsf(a)), "f"(fabsf(b)));
  return r;
}

// INT8 codes of a pair, as the low bytes of two words: what round_clamp_i8(x, s) gives, with
// r = fl(1 / s), without the IEEE division and without a conversion instruction in the common
// case.  |x| <= 127 (s - 1e-7), so t = fl(x * r) stays below 127.01 (no clamp needed) and within
// 128 * (2^-24 + 2^-24) < 1.6e-5 of x / s, whose correctly rounded value is within 7.7e-6 of it:
// when t is more than 1e-4 away from every half-integer, rint(t) equals rint(fl(x / s));
// otherwise (about one element in 5000) the division is done, after one test per eight elements.  rint(t) comes from adding
// 1.5 * 2^23: the sum is rounded to an integer (ties to even, like rint) and its low mantissa
// bits are that integer in two's complement, so the code is the low byte of the sum's bit
// pattern.  Packed FP32 instructions and byte permutes: about four instructions per element
// where conversions and shifts needed four times as many and bounded these kernels.
constexpr float kRoundMagic = 12582912.f;
__device__ __forceinline__ void round_i8_pair(float2 x, float2 r2, uint32_t& b0, uint32_t& b1, float& dmax) {
  const float2 t = __fmul2_rn(x, r2);
  const float2 tm = __fadd2_rn(t, make_float2(kRoundMagic, kRoundMagic));
  const float2 q = __fadd2_rn(tm, make_float2(-kRoundMagic, -kRoundMagic));
  const float2 d = __ffma2_rn(q, make_float2(-1.f, -1.f), t);  // t - q exactly, |d| <= 0.5
  b0 = __float_as_uint(tm.x);
  b1 = __float_as_uint(tm.y);
  dmax = absmax3(dmax, d.x, d.y);
}
// Eight elements of one row: codes in the low bytes of c[0..7].  One test per eight elements
// decides whether any of them is close to a half-integer; only then are those redone by division.
constexpr float kNearHalf = 0.4999f;
__device__ __forceinline__ void round_i8_row8(const float2 (&x)[4], float s, float r, uint32_t (&c)[8]) {
  const float2 r2 = make_float2(r, r);
  float dmax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) round_i8_pair(x[i], r2, c[2 * i], c[2 * i + 1], dmax);
  if (dmax > kNearHalf) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float tx = x[i].x * r, ty = x[i].y * r;
      if (fabsf(tx - rintf(tx)) > kNearHalf) c[2 * i] = static_cast<uint32_t>(round_clamp_i8(x[i].x, s));
      if (fabsf(ty - rintf(ty)) > kNearHalf) c[2 * i + 1] = static_cast<uint32_t>(round_clamp_i8(x[i].y, s));
    }
  }
}
// the low bytes of four words as one word
__device__ __forceinline__ uint32_t pack_low_bytes(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  return __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
}

// The work of kThreads threads (`tid` counts them) on NB consecutive 64-row blocks of head `bh`,
// starting at block `blk0`.  Every thread of the CTA must call it (it holds CTA-wide barriers);
// `row_max` and `row_scale` are this group's NB * 64 shared-memory slots.
// FULL: every row of the NB blocks exists (all CTAs of a head but the last): no per-row checks.
template <typename T, int D, bool IS_KEY, bool ALIGNED, int NB, bool FULL>
__device__ __forceinline__ void quantize_qk_body(
    const TensorArg& x, const float* __restrict__ mean, const int32_t* __restrict__ order, int8_t* __restrict__ codes,
    float* __restrict__ gscale, float* __restrict__ row_mul, int len, int len_pad, int heads, int per_thread,
    int groups_per_head, float mul, int bh, int blk0, int tid, float* row_max, float2* row_scale) {
  constexpr int TPR = D / 8;
  constexpr int RPP = kThreads / TPR;
  constexpr int NP = kBlockRows / RPP;
  const int cg = tid % TPR, rl = tid / TPR;
  const T* xp = static_cast<const T*>(head_ptr(x, bh, heads, sizeof(T)));

  float2 neg_mu[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    neg_mu[i] = IS_KEY ? make_float2(-mean[bh * D + cg * 8 + 2 * i], -mean[bh * D + cg * 8 + 2 * i + 1]) : make_float2(0.f, 0.f);

  // All row indices first, then all row loads, then the arithmetic: NB * NP 16-byte loads per
  // thread are in flight at once (two dependent levels when rows are gathered through `order`).
  // The rows stay in registers as loaded (four registers per load) and are unpacked twice, for
  // the abs-max and for the rounding step.
  Raw8<T> raw[NB][NP];
  int src[NB][NP];
#pragma unroll
  for (int b = 0; b < NB; ++b) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int r = (blk0 + b) * kBlockRows + p * RPP + rl;
      src[b][p] = -1;
      if (FULL || r < len) src[b][p] = (IS_KEY && order != nullptr) ? order[static_cast<long long>(bh) * len + r] : r;
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      if (FULL || src[b][p] >= 0) load8raw<T, ALIGNED>(xp + static_cast<long long>(src[b][p]) * x.ss + cg * 8, raw[b][p]);
      else raw[b][p].u = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  // One block per call: the unpacked (and smoothed) values stay in registers for the rounding
  // step.  More blocks: only the rows as loaded are kept and they are unpacked again.
  constexpr bool HOLD = NB == 1;
  float2 held[HOLD ? NP : 1][4];
#pragma unroll
  for (int b = 0; b < NB; ++b) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      float2 v[4];
      unpack8<T>(raw[b][p], v);
      float m = 0.f;
      if (FULL || src[b][p] >= 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (IS_KEY) v[i] = __fadd2_rn(v[i], neg_mu[i]);
          m = absmax3(m, v[i].x, v[i].y);
        }
      }
      if (HOLD) {
#pragma unroll
        for (int i = 0; i < 4; ++i) held[p][i] = v[i];
      }
      m = group_max<TPR>(m);
      if (cg == 0) row_max[b * kBlockRows + p * RPP + rl] = m;
    }
  }
  __syncthreads();
  if (tid < NB * kBlockRows) {  // two full warps per 64-row block: lane = row & 31
    const int r = tid % kBlockRows, blk = blk0 + tid / kBlockRows;
    const float own = row_max[tid], other = row_max[tid ^ 32];
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
    row_scale[tid] = make_float2(s, __fdiv_rn(1.f, s));
    const int gr = blk * kBlockRows + r;
    if (FULL || gr < len_pad) {
      row_mul[static_cast<long long>(bh) * len_pad + gr] = s * mul;
      if (per_thread) {
        if (FULL || gr < len) gscale[static_cast<long long>(bh) * groups_per_head + gr] = s;
      } else if (IS_KEY) {
        if (r == 0) gscale[static_cast<long long>(bh) * groups_per_head + blk] = s;
      } else if ((r & 31) == 0) {
        const int gi = blk * 2 + (r >> 5);
        if (gi < groups_per_head) gscale[static_cast<long long>(bh) * groups_per_head + gi] = s;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int b = 0; b < NB; ++b) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int lr = b * kBlockRows + p * RPP + rl;
      const int r = blk0 * kBlockRows + lr;
      if (!FULL && r >= len_pad) continue;
      const float2 sc = row_scale[lr];
      uint32_t c[8];
      if (HOLD) {
        round_i8_row8(held[p], sc.x, sc.y, c);
      } else {
        float2 v[4];
        unpack8<T>(raw[b][p], v);  // padding rows hold zeros and stay zero
        if (IS_KEY && (FULL || src[b][p] >= 0)) {
#pragma unroll
          for (int i = 0; i < 4; ++i) v[i] = __fadd2_rn(v[i], neg_mu[i]);
        }
        round_i8_row8(v, sc.x, sc.y, c);
      }
      *reinterpret_cast<uint2*>(codes + (static_cast<long long>(bh) * len_pad + r) * D + cg * 8) =
          make_uint2(pack_low_bytes(c[0], c[1], c[2], c[3]), pack_low_bytes(c[4], c[5], c[6], c[7]));
    }
  }
}

template <typename T, int D, bool IS_KEY, bool ALIGNED>
__global__ void __launch_bounds__(kThreads, 3) quantize_qk_kernel(
    TensorArg x, const float* __restrict__ mean, const int32_t* __restrict__ order, int8_t* __restrict__ codes,
    float* __restrict__ gscale, float* __restrict__ row_mul, int len, int len_pad, int heads, int per_thread,
    int groups_per_head, float mul) {
  cudaGridDependencySynchronize();  // launched chained: wait for the predecessor's writes
  // two blocks per CTA (eight 16-byte loads in flight per thread) measured 15 % faster than one
  // block with the unpacked values held, most of all for rows gathered through the key order
  __shared__ float row_max[kQuantBlocks * kBlockRows];
  __shared__ float2 row_scale[kQuantBlocks * kBlockRows];  // scale and its reciprocal
  const int blk0 = blockIdx.x * kQuantBlocks;
  if ((blk0 + kQuantBlocks) * kBlockRows <= len) {
    quantize_qk_body<T, D, IS_KEY, ALIGNED, kQuantBlocks, true>(x, mean, order, codes, gscale, row_mul, len, len_pad, heads,
                                                                per_thread, groups_per_head, mul, blockIdx.y, blk0,
                                                                threadIdx.x, row_max, row_scale);
  } else {
    quantize_qk_body<T, D, IS_KEY, ALIGNED, kQuantBlocks, false>(x, mean, order, codes, gscale, row_mul, len, len_pad, heads,
                                                                 per_thread, groups_per_head, mul, blockIdx.y, blk0,
                                                                 threadIdx.x, row_max, row_scale);
  }
}

// The key order of every head (CTAs [0, n_heads): one 1024-thread sort each, a few CTAs that
// run for a long time) and the Q quantisation (the other CTAs: four 256-thread groups, one
// 64-row block each) in one launch.  Neither depends on the other; launched apart, the sort
// would leave most of the GPU idle for as long as it runs.
template <typename T, int D, bool ALIGNED>
__global__ void __launch_bounds__(kSortThreads) sort_and_quantize_q_kernel(
    uint32_t* __restrict__ keys0, uint32_t* __restrict__ keys1, int32_t* __restrict__ idx0, int32_t* __restrict__ idx1,
    int n_keys, int n_heads, TensorArg q, int8_t* __restrict__ codes, float* __restrict__ gscale,
    float* __restrict__ row_mul, int len, int len_pad, int heads, int per_thread, int groups_per_head, float mul,
    int q_ctas_per_head) {
  cudaGridDependencySynchronize();  // launched chained: wait for the predecessor's writes
  constexpr int GROUPS = kSortThreads / kThreads;
  if (static_cast<int>(blockIdx.x) < n_heads) {
    segment_sort_body(keys0, keys1, idx0, idx1, n_keys, blockIdx.x);
  } else {
    __shared__ float row_max[GROUPS][kBlockRows];
    __shared__ float2 row_scale[GROUPS][kBlockRows];
    const int c = blockIdx.x - n_heads;
    const int bh = c / q_ctas_per_head, group = threadIdx.x / kThreads;
    const int blk0 = (c % q_ctas_per_head) * GROUPS + group;
    // the whole CTA takes one path (it holds CTA-wide barriers): the checked one unless all four blocks are full
    const int cta_last_row = ((c % q_ctas_per_head) * GROUPS + GROUPS) * kBlockRows;
    if (cta_last_row <= len) {
      quantize_qk_body<T, D, false, ALIGNED, 1, true>(q, nullptr, nullptr, codes, gscale, row_mul, len, len_pad, heads,
                                                      per_thread, groups_per_head, mul, bh, blk0, threadIdx.x % kThreads,
                                                      row_max[group], row_scale[group]);
    } else {
      quantize_qk_body<T, D, false, ALIGNED, 1, false>(q, nullptr, nullptr, codes, gscale, row_mul, len, len_pad, heads,
                                                       per_thread, groups_per_head, mul, bh, blk0, threadIdx.x % kThreads,
                                                       row_max[group], row_scale[group]);
    }
  }
}

// ---------------------------------------------------------------------------------------
// V quantisation.  Codes are written transposed, [head, feature, key], so that a 64-key tile
// is a K-major B operand of the PV product.  PIPER: per-key INT8 of (v - mean), plus
// log2(scale) and 1/scale per key.  SAGE: per-channel E4M3.
// ---------------------------------------------------------------------------------------
template <typename T, int D, bool SAGE, bool ALIGNED, bool FULL>
__device__ __forceinline__ void quantize_v_body(
    const TensorArg& v, const float* __restrict__ v_mean_or_scale, const int32_t* __restrict__ order,
    uint8_t* __restrict__ codes_t, float* __restrict__ v_scale, float* __restrict__ col_add,
    float* __restrict__ col_inv, int sk, int sk_pad, int heads, uint32_t* tile) {
  constexpr int TPR = D / 8;
  constexpr int RPP = kThreads / TPR;
  constexpr int NP = kBlockRows / RPP;  // adjacent keys per thread and block: 4 (head_dim 128) or 2 (64)
  constexpr int NB = kQuantBlocks;
  constexpr int WPR = NB * kBlockRows / 4;  // 32-bit words per feature row of the transposed tile
  static_assert(NP == 4 || NP == 2, "a thread's keys fill a word or half a word");
  // Transposed tile [feature][NB * 64 keys]; a thread owns NP adjacent keys of each 64-key block,
  // so it writes one (half) word per feature and block.  The word position is rotated by the
  // feature group so that the 16 (8) threads that hold the same keys of different feature
  // groups hit different banks.
  const int bh = blockIdx.y, blk0 = blockIdx.x * NB;
  const int cg = threadIdx.x % TPR, rl = threadIdx.x / TPR;
  const T* vp = static_cast<const T*>(head_ptr(v, bh, heads, sizeof(T)));

  float aux[8];  // PIPER: mean; SAGE: channel scale
#pragma unroll
  for (int i = 0; i < 8; ++i) aux[i] = v_mean_or_scale[bh * D + cg * 8 + i];

  // row indices, then all row loads (NB * NP 16-byte loads per thread in flight), then the arithmetic
  int src[NB][NP];
  Raw8<T> raw[NB][NP];
#pragma unroll
  for (int b = 0; b < NB; ++b) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int r = (blk0 + b) * kBlockRows + rl * NP + p;
      src[b][p] = -1;
      if (FULL || r < sk) src[b][p] = (!SAGE && order != nullptr) ? order[static_cast<long long>(bh) * sk + r] : r;
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      if (FULL || src[b][p] >= 0) load8raw<T, ALIGNED>(vp + static_cast<long long>(src[b][p]) * v.ss + cg * 8, raw[b][p]);
      else raw[b][p].u = make_uint4(0u, 0u, 0u, 0u);
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    uint32_t packed[8];  // per feature: this thread's NP adjacent keys of block b, one byte each
#pragma unroll
    for (int i = 0; i < 8; ++i) packed[i] = 0u;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int r = (blk0 + b) * kBlockRows + rl * NP + p;
      float2 x[4];
      unpack8<T>(raw[b][p], x);
      uint32_t c[8];  // word whose low byte is the code of (key p, feature i)
      if (!SAGE) {
        float m = 0.f;
        if (FULL || r < sk) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            x[i] = __fadd2_rn(x[i], make_float2(-aux[2 * i], -aux[2 * i + 1]));
            m = absmax3(m, x[i].x, x[i].y);
          }
        }
        m = group_max<TPR>(m);
        const float s = __fadd_rn(__fdiv_rn(m, 127.f), 1e-7f);
        const float rs = __fdiv_rn(1.f, s);
        if (cg == 0 && (FULL || r < sk_pad)) {
          const long long o = static_cast<long long>(bh) * sk_pad + r;
          if (FULL || r < sk) {
            v_scale[static_cast<long long>(bh) * sk + r] = s;
            col_add[o] = log2f(s);
            col_inv[o] = rs;
          } else {
            col_add[o] = -INFINITY;
            col_inv[o] = 0.f;
          }
        }
        round_i8_row8(x, s, rs, c);
      } else {
        if (cg == 0 && (FULL || r < sk_pad)) col_add[static_cast<long long>(bh) * sk_pad + r] = (FULL || r < sk) ? 0.f : -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          c[2 * i] = __nv_cvt_float_to_fp8(__fdiv_rn(x[i].x, aux[2 * i]), __NV_SATFINITE, __NV_E4M3);
          c[2 * i + 1] = __nv_cvt_float_to_fp8(__fdiv_rn(x[i].y, aux[2 * i + 1]), __NV_SATFINITE, __NV_E4M3);
        }
      }
      // byte p of packed[i] <- low byte of c[i]
      constexpr uint32_t kInsert[4] = {0x3214u, 0x3240u, 0x3410u, 0x4210u};
#pragma unroll
      for (int i = 0; i < 8; ++i) packed[i] = __byte_perm(packed[i], c[i], kInsert[p]);
    }
    const int key0 = b * kBlockRows + rl * NP;  // first of this thread's keys of block b within the tile
    const int word = ((key0 >> 2) + 4 * cg) % WPR;  // word position, rotated by four words per feature group
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t* row = tile + (cg * 8 + i) * WPR;
      if (NP == 4) row[word] = packed[i];
      else reinterpret_cast<uint16_t*>(row)[word * 2 + ((key0 >> 1) & 1)] = static_cast<uint16_t>(packed[i]);
    }
  }
  __syncthreads();
  // 16 bytes per thread and access: a feature's 128 keys are eight threads' stores (the rotation by
  // multiples of four words keeps each group of four words together)
  static_assert(WPR % 4 == 0 && (WPR & (WPR - 1)) == 0, "whole 16-byte groups per feature row");
  const int valid_quads = min(NB * kBlockRows, sk_pad - blk0 * kBlockRows) / 16;  // the last CTA may hold one block
  for (int idx = threadIdx.x; idx < D * (WPR / 4); idx += kThreads) {
    const int d = idx / (WPR / 4), g = idx % (WPR / 4);
    if (!FULL && g >= valid_quads) continue;
    const uint4 val = *reinterpret_cast<const uint4*>(tile + d * WPR + (4 * g + 4 * (d / 8)) % WPR);
    *reinterpret_cast<uint4*>(codes_t + (static_cast<long long>(bh) * D + d) * sk_pad + blk0 * kBlockRows + g * 16) = val;
  }
}

template <typename T, int D, bool SAGE, bool ALIGNED>
__global__ void __launch_bounds__(kThreads, 3) quantize_v_kernel(
    TensorArg v, const float* __restrict__ v_mean_or_scale, const int32_t* __restrict__ order,
    uint8_t* __restrict__ codes_t, float* __restrict__ v_scale, float* __restrict__ col_add,
    float* __restrict__ col_inv, int sk, int sk_pad, int heads) {
  cudaGridDependencySynchronize();  // launched chained: wait for the predecessor's writes
  __shared__ __align__(16) uint32_t tile[D * kQuantBlocks * kBlockRows / 4];
  // every key of this CTA's blocks exists (all CTAs of a head but the last): no per-key checks
  if ((static_cast<int>(blockIdx.x) + 1) * kQuantBlocks * kBlockRows <= sk) {
    quantize_v_body<T, D, SAGE, ALIGNED, true>(v, v_mean_or_scale, order, codes_t, v_scale, col_add, col_inv, sk, sk_pad, heads, tile);
  } else {
    quantize_v_body<T, D, SAGE, ALIGNED, false>(v, v_mean_or_scale, order, codes_t, v_scale, col_add, col_inv, sk, sk_pad, heads, tile);
  }
}

__global__ void zero_words_kernel(int32_t* p, int n) {
  cudaGridDependencySynchronize();  // launched chained: wait for the predecessor's writes
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

  launch_chained(zero_words_kernel, dim3(1), dim3(32), 0, st, at<int32_t>(p, L.status), 16);
  const bool do_kv = (parts & kPrepassKV) != 0, do_q = (parts & kPrepassQ) != 0;

  // With a key order to compute, the Q quantisation shares the launch of the sort (below).
  const bool q_with_sort = do_q && do_kv && sort;
  if (do_q && !q_with_sort) {
    launch_chained(quantize_qk_kernel<T, D, false, ALIGNED>, dim3(dim3(ceil_div(L.sq_pad / kBlockRows, kQuantBlocks), BH)), dim3(kThreads), 0, st, q, nullptr, nullptr, at<int8_t>(p, L.q_codes), at<float>(p, L.q_gscale), at<float>(p, L.q_mul), L.Sq,
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
    launch_chained(colstat_partial_kernel<T, D, ALIGNED>, dim3(dim3(L.chunks, BH)), dim3(kThreads), 0, st, k, v, at<double>(p, L.k_part), at<double>(p, L.v_part), L.Sk, p.heads, L.chunks, do_k, v_mode);
  }
  // v slot: piper -> mean [BH,D]; sage -> channel scale [BH,D] (stored in the v_scale view)
  float* v_stat = sage ? at<float>(p, L.v_scale) : at<float>(p, L.v_mean);
  const int fin_mode = sage ? 2 : (center ? 1 : 0);
  launch_chained(colstat_finalize_kernel, dim3(BH), dim3(2 * D), 0, st, at<double>(p, L.k_part), at<double>(p, L.v_part), p.k_mean_override,
                                            center ? p.v_mean_override : nullptr, at<float>(p, L.k_mean), v_stat,
                                            L.Sk, D, L.chunks, fin_mode);

  // 2. key order
  const int32_t* order = nullptr;
  if (sort) {
    constexpr int RPB = kRangePasses * (kThreads / (D / 8));  // rows per CTA
    launch_chained(row_range_kernel<T, D, ALIGNED>, dim3(dim3((L.Sk + RPB - 1) / RPB, BH)), dim3(kThreads), 0, st, v, at<float>(p, L.v_mean), at<uint32_t>(p, L.range), L.Sk, p.heads);
    if (q_with_sort) {
      const int q_ctas = ceil_div(L.sq_pad / kBlockRows, kSortThreads / kThreads);
      launch_chained(sort_and_quantize_q_kernel<T, D, ALIGNED>, dim3(BH + BH * q_ctas), dim3(kSortThreads), 0, st, at<uint32_t>(p, L.range), at<uint32_t>(p, L.keys_alt), at<int32_t>(p, L.idx_a), at<int32_t>(p, L.idx_b),
          L.Sk, BH, q, at<int8_t>(p, L.q_codes), at<float>(p, L.q_gscale), at<float>(p, L.q_mul), L.Sq, L.sq_pad,
          p.heads, per_thread, L.q_groups, p.scale * kLog2e, q_ctas);
    } else {
      launch_chained(segment_sort_kernel, dim3(BH), dim3(kSortThreads), 0, st, at<uint32_t>(p, L.range), at<uint32_t>(p, L.keys_alt),
                                                       at<int32_t>(p, L.idx_a), at<int32_t>(p, L.idx_b), L.Sk);
    }
    order = at<int32_t>(p, L.idx_a);
  }

  // 3. K codes
  launch_chained(quantize_qk_kernel<T, D, true, ALIGNED>, dim3(dim3(ceil_div(L.sk_pad / kBlockRows, kQuantBlocks), BH)), dim3(kThreads), 0, st, k, at<float>(p, L.k_mean), order, at<int8_t>(p, L.k_codes), at<float>(p, L.k_gscale), at<float>(p, L.k_mul),
      L.Sk, L.sk_pad, p.heads, per_thread, L.k_groups, 1.0f);

  // 4. V codes
  if (sage) {
    launch_chained(quantize_v_kernel<T, D, true, ALIGNED>, dim3(dim3(ceil_div(L.sk_pad / kBlockRows, kQuantBlocks), BH)), dim3(kThreads), 0, st, v, at<float>(p, L.v_scale), nullptr, at<uint8_t>(p, L.v_codes), nullptr, at<float>(p, L.k_add), nullptr,
        L.Sk, L.sk_pad, p.heads);
  } else {
    launch_chained(quantize_v_kernel<T, D, false, ALIGNED>, dim3(dim3(ceil_div(L.sk_pad / kBlockRows, kQuantBlocks), BH)), dim3(kThreads), 0, st, v, at<float>(p, L.v_mean), order, at<uint8_t>(p, L.v_codes), at<float>(p, L.v_scale), at<float>(p, L.k_add),
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
  if (al) launch_chained(colstat_partial_kernel<T, D, true>, dim3(dim3(chunks, BH)), dim3(kThreads), 0, st, k, v, k_part, v_part, p.kv_len, p.heads, chunks, 1, 1);
  else launch_chained(colstat_partial_kernel<T, D, false>, dim3(dim3(chunks, BH)), dim3(kThreads), 0, st, k, v, k_part, v_part, p.kv_len, p.heads, chunks, 1, 1);
  launch_chained(colstat_finalize_kernel, dim3(BH), dim3(2 * D), 0, st, k_part, v_part, nullptr, nullptr, k_mean, v_mean, p.kv_len, D, chunks, 1);
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
