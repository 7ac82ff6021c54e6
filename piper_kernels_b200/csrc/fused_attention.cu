// Fused quantized attention forward for sm_100a: piper_attention (INT8 QK^T, per-64-key
// UINT8 x INT8 PV with FP32 online softmax) and sage_attention_2pp (INT8 QK^T, E4M3 x E4M3 PV,
// FP16-rounded 64-key partials accumulated in FP32).
//
// Numerics follow the reference project's portable tile loop
//   src/piper_kernels/attention/piper/reference.py:93-156
//   src/piper_kernels/attention/sage2pp/reference.py:70-121
// with base-2 exponentials (log2(e) folded into the query multiplier) and the V row scale
// folded into the exponent: e_j = 2^(t_j - max_j t_j), t_j = score_j*log2e + log2(vscale_j),
// so the UINT8 code is rne(255*e_j) and the denominator term is e_j / vscale_j.
//
// One CTA owns a 128-row query tile of one (batch, head).  Warp roles:
//   softmax warpgroup(s)  thread = query row = tensor-memory lane; reads the INT32 score tile,
//                         writes the 8-bit probability tile back into tensor memory
//   dequant warpgroup     thread = query row; holds the FP32 numerator row, folds every 64-key
//                         PV partial into it, owns the running max / denominator, writes out
//   producer warp         TMA loads of the Q tile, K tiles, V^T tiles and per-key vectors
//   mma warp              one thread issues tcgen05.mma: S = Q K^T (SS form, kind::i8) and
//                         O_part = P V (A from tensor memory; kind::i8 U8xS8 or kind::f8f6f4)
// Piper's probability codes depend only on the tile's own maximum, so two softmax warpgroups
// process alternate key tiles in parallel; Sage's depend on the running maximum, so it uses one.
//
// Tensor memory (512 columns): four score buffers of 64 columns (the probability tile
// overwrites the first 16 columns of its score buffer), two PV-partial buffers of head_dim
// columns.  No cluster launch, no multicast; every wait is time-limited.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "pk_internal.h"
#include "pk_ptx.cuh"

namespace pk {
namespace {

constexpr int NK = 8;      // K tile ring
constexpr int NV = 4;      // V^T tile ring
constexpr int NVEC = 16;   // per-key vector ring (k_mul, k_add, k_inv: 3 x 64 floats)
constexpr int NSTAT = 8;   // softmax -> dequant per-row statistics ring
constexpr int NS = 4;      // score buffers in tensor memory
constexpr int NO = 2;      // PV partial buffers in tensor memory
constexpr int V_LAG = 4;   // the producer issues V^T tile j together with K tile j + V_LAG
constexpr int VEC_FLOATS = 3 * kKeyTile;
constexpr uint32_t TMEM_COLS = 512;
constexpr float kMagic = 12582912.f;  // 1.5 * 2^23: adding it rounds to an integer (ties to even)

struct FusedParams {
  const float* q_mul;   // [BH, sq_pad]
  const float* k_mul;   // [BH, sk_pad]
  const float* k_add;   // [BH, sk_pad]
  const float* k_inv;   // [BH, sk_pad]
  const float* v_aux;   // piper: V mean [BH, D]; sage: V channel scale [BH, D]
  void* out;
  int out_dtype;
  int Sq, Sk, sq_pad, sk_pad;
  int causal;
  int32_t* status;
  void* dump;
  int dump_bh, dump_qt;
};

template <int D, int ALGO>
struct Cfg {
  static constexpr int NSWG = (ALGO == kPiper) ? 2 : 1;
  static constexpr int THREADS = (NSWG + 2) * 128;
  static constexpr int Q_BYTES = kQTile * D;
  static constexpr int K_BYTES = kKeyTile * D;
  static constexpr int V_BYTES = D * kKeyTile;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + NK * K_BYTES;
  static constexpr int OFF_VEC = OFF_V + NV * V_BYTES;
  static constexpr int OFF_STAT = OFF_VEC + NVEC * VEC_FLOATS * 4;
  static constexpr int OFF_BAR = OFF_STAT + NSTAT * kQTile * 8;
  static constexpr int NUM_BARS = 1 + 2 * NK + 2 * NV + NVEC + 2 * NS + 2 * NO + NSTAT;
  static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;  // + slack for 1024-byte alignment
  static constexpr uint32_t COL_S = 0;
  static constexpr uint32_t COL_O = NS * kKeyTile;
};

// barrier indices
struct Bars {
  uint32_t base;
  __device__ uint32_t q_full() const { return base; }
  __device__ uint32_t k_full(int i) const { return base + 8 * (1 + i); }
  __device__ uint32_t k_empty(int i) const { return base + 8 * (1 + NK + i); }
  __device__ uint32_t v_full(int i) const { return base + 8 * (1 + 2 * NK + i); }
  __device__ uint32_t v_empty(int i) const { return base + 8 * (1 + 2 * NK + NV + i); }
  __device__ uint32_t vec_full(int i) const { return base + 8 * (1 + 2 * NK + 2 * NV + i); }
  __device__ uint32_t s_full(int i) const { return base + 8 * (1 + 2 * NK + 2 * NV + NVEC + i); }
  __device__ uint32_t p_ready(int i) const { return base + 8 * (1 + 2 * NK + 2 * NV + NVEC + NS + i); }
  __device__ uint32_t o_full(int i) const { return base + 8 * (1 + 2 * NK + 2 * NV + NVEC + 2 * NS + i); }
  __device__ uint32_t o_empty(int i) const { return base + 8 * (1 + 2 * NK + 2 * NV + NVEC + 2 * NS + NO + i); }
  __device__ uint32_t stat_full(int i) const {
    return base + 8 * (1 + 2 * NK + 2 * NV + NVEC + 2 * NS + 2 * NO + i);
  }
};

// wait-site codes reported in status[0] when a wait is abandoned
enum : int {
  W_PROD_K = 11, W_PROD_V = 12, W_MMA_Q = 21, W_MMA_K = 22, W_MMA_P = 23, W_MMA_O = 24, W_MMA_V = 25,
  W_SM_VEC = 31, W_SM_S = 32, W_DQ_STAT = 41, W_DQ_O = 42
};

__device__ __forceinline__ float round_through_f16(float x) { return __half2float(__float2half_rn(x)); }

template <int D, int ALGO, bool K_PER_BLOCK>
__global__ void __launch_bounds__(Cfg<D, ALGO>::THREADS, 1)
fused_attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const FusedParams prm) {
  using C = Cfg<D, ALGO>;
  constexpr int NSWG = C::NSWG;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const Bars bars{smem_base + C::OFF_BAR};
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 4);
  float* vec_ring = reinterpret_cast<float*>(smem + C::OFF_VEC);
  float2* stat_ring = reinterpret_cast<float2*>(smem + C::OFF_STAT);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, wg = warp >> 2;
  const int bh = blockIdx.y;
  const int n_qt = prm.sq_pad / kQTile;
  const int qt = prm.causal ? (n_qt - 1 - blockIdx.x) : blockIdx.x;  // causal: longest tiles first
  const int q0 = qt * kQTile;
  const int n_all = prm.sk_pad / kKeyTile;
  const int n_tiles = prm.causal ? min(n_all, 2 * qt + 2) : n_all;
  const bool dumping = prm.dump != nullptr && bh == prm.dump_bh && qt == prm.dump_qt;

  if (tid == 0) {
    mbar_init(bars.q_full(), 1);
    for (int i = 0; i < NK; ++i) { mbar_init(bars.k_full(i), 1); mbar_init(bars.k_empty(i), 1); }
    for (int i = 0; i < NV; ++i) { mbar_init(bars.v_full(i), 1); mbar_init(bars.v_empty(i), 1); }
    for (int i = 0; i < NVEC; ++i) mbar_init(bars.vec_full(i), 1);
    for (int i = 0; i < NS; ++i) { mbar_init(bars.s_full(i), 1); mbar_init(bars.p_ready(i), 128); }
    for (int i = 0; i < NO; ++i) { mbar_init(bars.o_full(i), 1); mbar_init(bars.o_empty(i), 128); }
    for (int i = 0; i < NSTAT; ++i) mbar_init(bars.stat_full(i), 128);
    *abort_flag = 0;
    fence_barrier_init();
  }
  constexpr int PROD_WARP = (NSWG + 1) * 4;
  constexpr int MMA_WARP = PROD_WARP + 1;
  if (warp == PROD_WARP) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The CTA starts with 128 (piper, 512 threads) or 168 (sage, 384 threads) registers per
  // thread; the dequant rows need more and the helper warpgroup far fewer, so each role
  // resizes its allocation on entry.
  if (wg == NSWG + 1) {
    setmaxnreg_dec<24>();
  }
  if (warp == PROD_WARP) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v);
      mbar_expect_tx(bars.q_full(), C::Q_BYTES);
      tma_load_2d(smem_base + C::OFF_Q, &tm_q, bars.q_full(), 0, bh * prm.sq_pad + q0);
      const long long vec_base = static_cast<long long>(bh) * prm.sk_pad;
      for (int i = 0; i < n_tiles + V_LAG; ++i) {
        if (i < n_tiles) {
          const int s = i % NK;
          if (i >= NK && !mbar_wait_bounded(bars.k_empty(s), ((i / NK) - 1) & 1, abort_flag, W_PROD_K)) break;
          mbar_expect_tx(bars.k_full(s), C::K_BYTES);
          tma_load_2d(smem_base + C::OFF_K + s * C::K_BYTES, &tm_k, bars.k_full(s), 0,
                      bh * prm.sk_pad + i * kKeyTile);
          // The vector slot of tile i-NVEC was last read before the PV product of that tile was
          // issued, which precedes the release of the K stage waited for above.
          const int vs = i % NVEC;
          const uint32_t vdst = smem_base + C::OFF_VEC + vs * VEC_FLOATS * 4;
          mbar_expect_tx(bars.vec_full(vs), VEC_FLOATS * 4);
          const long long off = vec_base + static_cast<long long>(i) * kKeyTile;
          bulk_load(vdst, prm.k_mul + off, kKeyTile * 4, bars.vec_full(vs));
          bulk_load(vdst + kKeyTile * 4, prm.k_add + off, kKeyTile * 4, bars.vec_full(vs));
          bulk_load(vdst + 2 * kKeyTile * 4, prm.k_inv + off, kKeyTile * 4, bars.vec_full(vs));
        }
        const int j = i - V_LAG;
        if (j >= 0 && j < n_tiles) {
          const int s = j % NV;
          if (j >= NV && !mbar_wait_bounded(bars.v_empty(s), ((j / NV) - 1) & 1, abort_flag, W_PROD_V)) break;
          mbar_expect_tx(bars.v_full(s), C::V_BYTES);
          tma_load_2d(smem_base + C::OFF_V + s * C::V_BYTES, &tm_v, bars.v_full(s), j * kKeyTile, bh * D);
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------------ mma issue
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(kAccS32, kFmtS8, kFmtS8, kQTile, kKeyTile);
      constexpr uint32_t idesc_pv = (ALGO == kPiper) ? umma_idesc(kAccS32, kFmtU8, kFmtS8, kQTile, D)
                                                     : umma_idesc(kAccF32, kFmtE4M3, kFmtE4M3, kQTile, D);
      const uint64_t qdesc = umma_smem_desc(smem_base + C::OFF_Q, D);
      bool ok = mbar_wait_bounded(bars.q_full(), 0, abort_flag, W_MMA_Q);
      auto issue_qk = [&](int j) -> bool {
        const int s = j % NK;
        if (!mbar_wait_bounded(bars.k_full(s), (j / NK) & 1, abort_flag, W_MMA_K)) return false;
        tc_fence_after();
        const uint64_t kdesc = umma_smem_desc(smem_base + C::OFF_K + s * C::K_BYTES, D);
        const uint32_t d = tmem_base + C::COL_S + (j % NS) * kKeyTile;
#pragma unroll
        for (int kk = 0; kk < D / 32; ++kk) umma_i8_ss(d, qdesc + 2 * kk, kdesc + 2 * kk, idesc_qk, kk > 0);
        tc_commit(bars.s_full(j % NS));
        tc_commit(bars.k_empty(s));
        return true;
      };
      for (int j = 0; ok && j < min(NS, n_tiles); ++j) ok = issue_qk(j);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (!mbar_wait_bounded(bars.p_ready(j % NS), (j / NS) & 1, abort_flag, W_MMA_P)) break;
        if (j >= NO && !mbar_wait_bounded(bars.o_empty(j % NO), ((j / NO) - 1) & 1, abort_flag, W_MMA_O)) break;
        const int s = j % NV;
        if (!mbar_wait_bounded(bars.v_full(s), (j / NV) & 1, abort_flag, W_MMA_V)) break;
        tc_fence_after();
        const uint64_t vdesc = umma_smem_desc(smem_base + C::OFF_V + s * C::V_BYTES, kKeyTile);
        const uint32_t d = tmem_base + C::COL_O + (j % NO) * D;
        const uint32_t a = tmem_base + C::COL_S + (j % NS) * kKeyTile;
#pragma unroll
        for (int kk = 0; kk < kKeyTile / 32; ++kk) {
          if (ALGO == kPiper) umma_i8_ts(d, a + 8 * kk, vdesc + 2 * kk, idesc_pv, kk > 0);
          else umma_f8_ts(d, a + 8 * kk, vdesc + 2 * kk, idesc_pv, kk > 0);
        }
        tc_commit(bars.o_full(j % NO));
        tc_commit(bars.v_empty(s));
        if (j + NS < n_tiles) ok = issue_qk(j + NS);
      }
    }
  } else if (wg < NSWG) {
    // ------------------------------------------------------------------ softmax
    if (NSWG == 2) setmaxnreg_inc<152>(); else setmaxnreg_dec<160>();
    const int row = tid & 127;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const float qm = prm.q_mul[static_cast<long long>(bh) * prm.sq_pad + q0 + row];
    float m_run = -INFINITY;  // sage only
    for (int j = wg; j < n_tiles; j += NSWG) {
      // votes keep the warp converged for the .sync.aligned tensor-memory ops even when a wait is abandoned
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bars.vec_full(j % NVEC), (j / NVEC) & 1, abort_flag, W_SM_VEC))) break;
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bars.s_full(j % NS), (j / NS) & 1, abort_flag, W_SM_S))) break;
      tc_fence_after();
      const uint32_t s_addr = lane_addr + C::COL_S + (j % NS) * kKeyTile;
      uint32_t sraw[kKeyTile];
      tmem_ld32(s_addr, sraw);
      tmem_ld32(s_addr + 32, sraw + 32);
      tmem_wait_ld();
      if (dumping && j == 0) {
        int32_t* ds = static_cast<int32_t*>(prm.dump);
#pragma unroll
        for (int c = 0; c < kKeyTile; ++c) ds[row * kKeyTile + c] = static_cast<int32_t>(sraw[c]);
      }
      const float4* vk = reinterpret_cast<const float4*>(vec_ring + (j % NVEC) * VEC_FLOATS);
      float t[kKeyTile];
      const float mt = K_PER_BLOCK ? qm * vec_ring[(j % NVEC) * VEC_FLOATS] : 0.f;
#pragma unroll
      for (int c4 = 0; c4 < kKeyTile / 4; ++c4) {
        const float4 add = vk[kKeyTile / 4 + c4];
        const float a4[4] = {add.x, add.y, add.z, add.w};
        float m4[4] = {mt, mt, mt, mt};
        if (!K_PER_BLOCK) {
          const float4 mul = vk[c4];
          m4[0] = mul.x; m4[1] = mul.y; m4[2] = mul.z; m4[3] = mul.w;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float sf = static_cast<float>(static_cast<int32_t>(sraw[c4 * 4 + i]));
          t[c4 * 4 + i] = K_PER_BLOCK ? fmaf(sf, m4[i], a4[i]) : fmaf(sf * qm, m4[i], a4[i]);
        }
      }
      if (prm.causal && j * kKeyTile + kKeyTile - 1 > q0) {
        const int lim = q0 + row - j * kKeyTile;  // columns above this index are masked
#pragma unroll
        for (int c = 0; c < kKeyTile; ++c)
          if (c > lim) t[c] = -INFINITY;
      }
      float bm = t[0];
#pragma unroll
      for (int c = 1; c < kKeyTile; ++c) bm = fmaxf(bm, t[c]);

      uint32_t packed[kKeyTile / 4];
      float2 st;
      if (ALGO == kPiper) {
        const float bs = (bm == -INFINITY) ? 0.f : bm;
        float psum = 0.f;
#pragma unroll
        for (int c4 = 0; c4 < kKeyTile / 4; ++c4) {
          const float4 inv = vk[2 * (kKeyTile / 4) + c4];
          const float i4[4] = {inv.x, inv.y, inv.z, inv.w};
          uint32_t b[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float e = ex2_approx(t[c4 * 4 + i] - bs);
            psum = fmaf(e, i4[i], psum);
            b[i] = __float_as_uint(fmaf(e, 255.f, kMagic));  // low byte = rne(255 e)
          }
          const uint32_t lo = __byte_perm(b[0], b[1], 0x0040);
          const uint32_t hi = __byte_perm(b[2], b[3], 0x0040);
          packed[c4] = __byte_perm(lo, hi, 0x5410);
        }
        st = make_float2(bm, psum);
      } else {
        const float nm = fmaxf(m_run, bm);
        const float ns = (nm == -INFINITY) ? 0.f : nm;
        const float ow = (m_run == nm) ? 1.f : ex2_approx(m_run - ns);
        const float off = ns - 8.807354922057604f;  // log2(448): P = e4m3(448 * 2^(t - max))
        float psum = 0.f;
#pragma unroll
        for (int c4 = 0; c4 < kKeyTile / 4; ++c4) {
          float e[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            e[i] = ex2_approx(t[c4 * 4 + i] - off);
            psum += e[i];
          }
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(e[0], e[1]), __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(e[2], e[3]), __NV_SATFINITE, __NV_E4M3);
          packed[c4] = lo | (hi << 16);
        }
        st = make_float2(ow, psum * (1.f / 448.f));
        m_run = nm;
      }
      tmem_st16(s_addr, packed);
      tmem_wait_st();
      stat_ring[(j % NSTAT) * kQTile + row] = st;
      if (dumping && j == 0) {
        uint32_t* dp = reinterpret_cast<uint32_t*>(static_cast<char*>(prm.dump) + kQTile * kKeyTile * 4);
#pragma unroll
        for (int c = 0; c < kKeyTile / 4; ++c) dp[row * (kKeyTile / 4) + c] = packed[c];
      }
      tc_fence_before();
      mbar_arrive(bars.p_ready(j % NS));
      mbar_arrive(bars.stat_full(j % NSTAT));
    }
  } else if (wg == NSWG) {
    // ------------------------------------------------------------------ dequant + epilogue
    if (NSWG == 2) setmaxnreg_inc<184>(); else setmaxnreg_inc<216>();
    const int row = tid & 127;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    float num[D];
#pragma unroll
    for (int d = 0; d < D; ++d) num[d] = 0.f;
    float den = 0.f, m = -INFINITY;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bars.stat_full(j % NSTAT), (j / NSTAT) & 1, abort_flag, W_DQ_STAT))) { ok = false; break; }
      const float2 st = stat_ring[(j % NSTAT) * kQTile + row];
      float ow, c;
      if (ALGO == kPiper) {
        const float bm = st.x;
        const float nm = fmaxf(m, bm);
        float cw;
        if (nm == -INFINITY) { ow = 1.f; cw = 0.f; }
        else {
          ow = (m == nm) ? 1.f : ex2_approx(m - nm);
          cw = (bm == nm) ? 1.f : ex2_approx(bm - nm);
        }
        den = fmaf(den, ow, st.y * cw);
        c = __fdiv_rn(cw, 255.f);
        m = nm;
      } else {
        ow = st.x;
        den = fmaf(den, ow, st.y);
        c = 1.f;
      }
      if (!__all_sync(0xffffffffu, mbar_wait_bounded(bars.o_full(j % NO), (j / NO) & 1, abort_flag, W_DQ_O))) { ok = false; break; }
      tc_fence_after();
      if (__any_sync(0xffffffffu, ow != 1.f)) {
#pragma unroll
        for (int d = 0; d < D; ++d) num[d] *= ow;
      }
      const uint32_t o_addr = lane_addr + C::COL_O + (j % NO) * D;
#pragma unroll
      for (int ch = 0; ch < D / 32; ++ch) {
        uint32_t o[32];
        tmem_ld32(o_addr + ch * 32, o);
        tmem_wait_ld();
        if (dumping && j == 0) {
          uint32_t* dp = reinterpret_cast<uint32_t*>(static_cast<char*>(prm.dump) + kQTile * kKeyTile * 5);
#pragma unroll
          for (int i = 0; i < 32; ++i) dp[row * D + ch * 32 + i] = o[i];
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (ALGO == kPiper) num[ch * 32 + i] = fmaf(static_cast<float>(static_cast<int32_t>(o[i])), c, num[ch * 32 + i]);
          else num[ch * 32 + i] += round_through_f16(__uint_as_float(o[i]));
        }
      }
      tc_fence_before();
      mbar_arrive(bars.o_empty(j % NO));
    }
    // epilogue: normalise, restore the V mean (piper) / apply the channel scale (sage), cast
    const int grow = q0 + row;
    if (ok && grow < prm.Sq) {
      const float dmax = fmaxf(den, 1e-30f);
      const float* aux = prm.v_aux + static_cast<long long>(bh) * D;
      const long long obase = (static_cast<long long>(bh) * prm.Sq + grow) * D;
#pragma unroll
      for (int d0 = 0; d0 < D; d0 += 8) {
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (ALGO == kPiper) r[i] = __fdiv_rn(num[d0 + i], dmax) + aux[d0 + i];
          else r[i] = __fdiv_rn(num[d0 + i] * __fdiv_rn(aux[d0 + i], 448.f), dmax);
        }
        if (prm.out_dtype == PK_F32) {
          float4* o = reinterpret_cast<float4*>(static_cast<float*>(prm.out) + obase + d0);
          o[0] = make_float4(r[0], r[1], r[2], r[3]);
          o[1] = make_float4(r[4], r[5], r[6], r[7]);
        } else {
          uint32_t w[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (prm.out_dtype == PK_F16) {
              const __half2 h = __floats2half2_rn(r[2 * i], r[2 * i + 1]);
              w[i] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
              const __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * i], r[2 * i + 1]);
              w[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
          }
          *reinterpret_cast<uint4*>(static_cast<uint16_t*>(prm.out) + obase + d0) = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == PROD_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (tid == 0 && *abort_flag != 0) atomicCAS(prm.status, 0, *abort_flag);
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// 2-D byte tensor [rows, cols] (cols contiguous), box [box_rows, box_cols], swizzle = box_cols bytes.
int make_map(CUtensorMap* m, void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(PK_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = box_cols == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(PK_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return PK_OK;
}

template <int D, int ALGO, bool KPB>
int launch_one(const pk_problem& p, const Layout& L, cudaStream_t st, const DebugDump* dump) {
  using C = Cfg<D, ALGO>;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_map(&tq, at<void>(p, L.q_codes), static_cast<uint64_t>(L.BH) * L.sq_pad, D, kQTile, D))) return rc;
  if ((rc = make_map(&tk, at<void>(p, L.k_codes), static_cast<uint64_t>(L.BH) * L.sk_pad, D, kKeyTile, D))) return rc;
  if ((rc = make_map(&tv, at<void>(p, L.v_codes), static_cast<uint64_t>(L.BH) * D, L.sk_pad, D, kKeyTile))) return rc;
  FusedParams prm{};
  prm.q_mul = at<float>(p, L.q_mul);
  prm.k_mul = at<float>(p, L.k_mul);
  prm.k_add = at<float>(p, L.k_add);
  prm.k_inv = at<float>(p, L.k_inv);
  prm.v_aux = ALGO == kPiper ? at<float>(p, L.v_mean) : at<float>(p, L.v_scale);
  prm.out = p.out;
  prm.out_dtype = p.out_dtype;
  prm.Sq = L.Sq; prm.Sk = L.Sk; prm.sq_pad = L.sq_pad; prm.sk_pad = L.sk_pad;
  prm.causal = p.is_causal;
  prm.status = at<int32_t>(p, L.status);
  prm.dump = dump ? dump->ptr : nullptr;
  prm.dump_bh = dump ? dump->bh : -1;
  prm.dump_qt = dump ? dump->q_tile : -1;
  auto kern = fused_attention_kernel<D, ALGO, KPB>;
  {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    if (e != cudaSuccess) return fail(PK_ERR_CUDA, "cudaFuncSetAttribute: %s", cuda_err(e));
  }
  const dim3 grid(L.sq_pad / kQTile, L.BH);
  kern<<<grid, C::THREADS, C::SMEM_BYTES, st>>>(tq, tk, tv, prm);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PK_ERR_CUDA, "fused kernel launch failed: %s", cuda_err(e));
  return PK_OK;
}

template <int D, int ALGO>
int launch_gran(const pk_problem& p, const Layout& L, cudaStream_t st, const DebugDump* dump) {
  return p.qk_granularity == PK_QK_PER_BLOCK ? launch_one<D, ALGO, true>(p, L, st, dump)
                                             : launch_one<D, ALGO, false>(p, L, st, dump);
}

}  // namespace

int launch_fused(const pk_problem& p, const Layout& L, Algo algo, cudaStream_t st, const DebugDump* dump) {
  if (algo == kPiper) return p.head_dim == 128 ? launch_gran<128, kPiper>(p, L, st, dump) : launch_gran<64, kPiper>(p, L, st, dump);
  return p.head_dim == 128 ? launch_gran<128, kSage>(p, L, st, dump) : launch_gran<64, kSage>(p, L, st, dump);
}

}  // namespace pk
