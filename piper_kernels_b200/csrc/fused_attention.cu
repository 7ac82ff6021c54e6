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
//                         writes the 8-bit probability tile into tensor memory
//   dequant warpgroup     thread = query row; holds the FP32 numerator row, folds every 64-key
//                         PV partial into it, owns the running max / denominator, writes out
//   producer warp         TMA loads of the Q tile, K tiles, V^T tiles and per-key vectors
//   two issue warps       tcgen05.mma: S = Q K^T (SS form, kind::i8) and O_part = P V (A from
//                         tensor memory; kind::i8 U8xS8 or kind::f8f6f4)
// The three helper warps run their loops and waits with all lanes and issue from the lane that
// elect.sync picks.
// Two softmax warpgroups process alternate key tiles.  Piper's probability codes depend only on
// the tile's own maximum; Sage's depend on the running maximum, which one warpgroup hands to the
// other through shared memory as soon as it knows its tile's maximum, so that only this short
// step is sequential and the exponentials of consecutive tiles overlap.
//
// INT32 accumulators are read as FP32 without an integer instruction: every INT32 buffer is
// re-armed with the bit pattern of 1.5*2^23 by the warp that has just read it, and the next
// product accumulates on top, so the word read back is the float 1.5*2^23 + value exactly
// (|value| < 2^22); one packed FP32 subtract recovers the value.
//
// Tensor memory (512 columns): three score buffers of 64 columns, four probability buffers
// of 16 columns, two PV-partial buffers of head_dim columns.  No cluster launch, no
// multicast; every wait is time-limited.

#include <cuda.h>

#include <atomic>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "pk_internal.h"
#include "pk_ptx.cuh"

// Votes keep a warp converged around the .sync.aligned tensor-memory instructions when a wait is
// abandoned.
#define WARP_ALL(x) __all_sync(0xffffffffu, (x))
#define WARP_ANY(x) __any_sync(0xffffffffu, (x))
// A helper warp (producer, S issue, PV issue) runs its loop either with lane 0 alone or with all
// 32 lanes, issuing from the lane elect.sync picks.  HCONV says which for the role being
// compiled (HROLE_CONVERGED is set in front of each role), HLANE admits the lanes that run the
// loop, HWAIT wraps a wait, HELECT guards the issuing instructions.
#define HCONV (HROLE_CONVERGED)
#define HLANE (HCONV || lane == 0)
#define HWAIT(x) (HCONV ? WARP_ALL(x) : (x))
#define HELECT (HCONV ? elect_one() : true)
namespace pk {
namespace {

constexpr int NK = 8;      // K tile ring
constexpr int NV = 8;      // V^T tile ring (a copy from L2 takes longer than four tiles last)
constexpr int NVEC = 16;   // per-key vector ring (k_mul, k_add, k_inv: 3 x 64 floats)
constexpr int NSTAT = 8;   // softmax -> dequant per-row statistics ring
constexpr int NM = 4;      // sage: running-maximum hand-over ring between the two softmax warpgroups
constexpr int NS = 3;      // score buffers in tensor memory
constexpr int NP = 4;      // probability buffers in tensor memory
constexpr int NO = 2;      // PV partial buffers in tensor memory
constexpr int NPV = NV;    // completion barriers of the PV products: one per V stage (a multiple of NP)
constexpr int VEC_FLOATS = 3 * kKeyTile;
constexpr uint32_t TMEM_COLS = 512;
constexpr int kPrefetchCtasAhead = 160;  // a little more than one CTA per SM
constexpr float kMagic = 12582912.f;    // 1.5 * 2^23: adding it rounds to an integer (ties to even)
constexpr uint32_t kMagicBits = 0x4B400000u;  // bit pattern of kMagic

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
  long long* timeline;  // optional [6][timeline_tiles][4] clock stamps of CTA (dump_bh, dump_qt)
  int timeline_tiles;
  int splits, tiles_per_split;  // key split of small problems (1: none); CTA z handles tiles [z*tps, (z+1)*tps)
  float* partial;               // [BH, sq_pad, splits, D + 4] numerators, running max, denominator (splits > 1)
  int skip_key_tile;        // stalled-wait drill only: key tile whose copy the producer leaves out
  int32_t* host_status;     // optional pinned host word (device-visible) that also receives the code
};

template <int D, int ALGO>
struct Cfg {
  static constexpr int NSWG = 2;  // softmax warpgroups, on alternate key tiles
  static constexpr int NDQ = 1;   // dequant warpgroup
  static constexpr int THREADS = (NSWG + NDQ + 1) * 128;         // + the helper warpgroup
  static constexpr int LAUNCH_REGS = (65536 / THREADS) / 8 * 8;  // 128 registers per thread at launch
  // Per-role register budgets (setmaxnreg): the dequant rows hold head_dim FP32 numerators each.
  static constexpr bool SAGE64 = ALGO == kSage && D == 64;
  static constexpr int REG_SM = SAGE64 ? 152 : 120;
  static constexpr int REG_DQ = SAGE64 ? 144 : 232;
  static constexpr int REG_HELPER = SAGE64 ? 56 : 40;
  // The two issue warps run converged and issue from the lane elect.sync picks: the compiler then
  // keeps descriptors and addresses in uniform registers (47 instead of about 80 cycles per issued
  // product).  The producer does the same for sage; for piper at long key sequences it measured
  // 1-2 % faster with lane 0 running the loop alone.
  static constexpr bool PRODUCER_CONVERGED = ALGO == kSage;
  static constexpr int PRODUCER_SLEEP_NS = ALGO == kPiper ? 500 : 0;
  // Where the dequant warpgroup evaluates a tile's factors and waits for its product: at the top
  // of the tile (the eight chunks of the fold are then one straight-line block that the compiler
  // schedules as a whole: 6-7 % faster for piper, where the dequant sets the period), or one tile
  // ahead in the middle of the previous tile's fold with the first chunk's load in flight across
  // the tile boundary (1 % faster for sage at head_dim 64, where the softmax warpgroups set it).
  static constexpr bool FOLD_FROM_TILE_TOP = !(ALGO == kSage && D == 64);
  // setmaxnreg only moves registers between the warps of the CTA: an increase waits (without a time
  // limit) until other warps have released enough, so the budgets must fit what the CTA was launched with.
  static_assert((NSWG * REG_SM + NDQ * REG_DQ + REG_HELPER) * 128 <= THREADS * LAUNCH_REGS,
                "role register budgets exceed the registers the CTA owns");
  static constexpr int Q_BYTES = kQTile * D;
  static constexpr int K_BYTES = kKeyTile * D;
  static constexpr int V_BYTES = D * kKeyTile;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + NK * K_BYTES;
  static constexpr int OFF_VEC = OFF_V + NV * V_BYTES;
  static constexpr int OFF_STAT = OFF_VEC + NVEC * VEC_FLOATS * 4;
  static constexpr int OFF_MRING = OFF_STAT + NSTAT * kQTile * 8;
  static constexpr int OFF_BAR = OFF_MRING + NM * kQTile * 4;
  static constexpr int NUM_BARS = 1 + 2 * NK + NV + NVEC + NS + NP + NPV + NO + NSTAT + NM;
  static constexpr int OFF_MISC = (OFF_BAR + NUM_BARS * 8 + 15) / 16 * 16;
  static constexpr int OFF_MAGIC = OFF_MISC + 16;           // 16 words holding the arming pattern
  static constexpr int OFF_AUX = OFF_MAGIC + 64;            // head_dim floats: V mean (piper) / V channel scale (sage)
  static constexpr int SMEM_BYTES = OFF_AUX + D * 4 + 1024;  // + slack for 1024-byte alignment
  static constexpr uint32_t COL_S = 0;
  static constexpr uint32_t COL_P = NS * kKeyTile;
  static constexpr uint32_t COL_O = COL_P + NP * (kKeyTile / 4);
  static_assert(COL_O + NO * D <= TMEM_COLS, "tensor memory budget");
  static_assert(OFF_MAGIC % 16 == 0, "the arming block is read with 16-byte loads");
};

// shared-memory addresses of the mbarriers.  One commit per product: qk_done[j % NK] is
// observed by the softmax warpgroup (scores ready) and by the producer (K stage free);
// pv_done[j % NPV] by the dequant warpgroup (partial ready), the producer (V stage free) and
// the softmax warpgroup (probability buffer free).
struct Bars {
  uint32_t base;
  __device__ uint32_t at(int i) const { return base + 8 * i; }
  __device__ uint32_t q_full() const { return at(0); }
  __device__ uint32_t k_full(int i) const { return at(1 + i); }
  __device__ uint32_t qk_done(int i) const { return at(1 + NK + i); }
  __device__ uint32_t v_full(int i) const { return at(1 + 2 * NK + i); }
  __device__ uint32_t vec_full(int i) const { return at(1 + 2 * NK + NV + i); }
  __device__ uint32_t s_free(int i) const { return at(1 + 2 * NK + NV + NVEC + i); }
  __device__ uint32_t p_ready(int i) const { return at(1 + 2 * NK + NV + NVEC + NS + i); }
  __device__ uint32_t pv_done(int i) const { return at(1 + 2 * NK + NV + NVEC + NS + NP + i); }
  __device__ uint32_t o_empty(int i) const { return at(1 + 2 * NK + NV + NVEC + NS + NP + NPV + i); }
  __device__ uint32_t stat_full(int i) const { return at(1 + 2 * NK + NV + NVEC + NS + NP + NPV + NO + i); }
  __device__ uint32_t m_ready(int i) const { return at(1 + 2 * NK + NV + NVEC + NS + NP + NPV + NO + NSTAT + i); }
};
static_assert(NPV == NV && NPV % NP == 0 && NPV >= NP,
              "pv_done[t % NPV] tells the producer that V stage t % NV is free, the softmax warpgroups that "
              "probability buffer t % NP is free and the dequant warpgroup that partial t is complete");

// wait-site codes reported in status[0] when a wait is abandoned
enum : int {
  W_PROD_K = 11, W_PROD_V = 12, W_QK_Q = 21, W_QK_K = 22, W_QK_S = 23, W_PV_P = 26, W_PV_O = 27, W_PV_V = 28,
  W_SM_VEC = 31, W_SM_S = 32, W_SM_PV = 33, W_SM_M = 34, W_DQ_STAT = 41, W_DQ_O = 42
};

// Per-role timeline of one CTA for pk_debug_timeline(): int64 clock64() stamps laid out
// [role][tile][8], roles: the softmax warpgroups first (two at head_dim 128, three at 64), then
// dequant, S-product issue, PV-product issue; at most 7 roles.  One thread per role stamps; other
// CTAs and ordinary launches skip it.
#define PK_STAMP(role, tile, k)                                                                     \
  do {                                                                                               \
    if (TIMELINE && stamping && (tile) < prm.timeline_tiles)                                         \
      prm.timeline[(static_cast<long long>(role) * prm.timeline_tiles + (tile)) * 8 + (k)] = clock64(); \
  } while (0)

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Stores the magic bit pattern into `ncols` (multiple of 16) columns of this thread's lane.
__device__ __forceinline__ void tmem_arm(uint32_t addr, int ncols) {
  uint32_t m[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) m[i] = kMagicBits;
  for (int c = 0; c < ncols; c += 16) tmem_st16(addr + c, m);
}

// Sixteen registers holding the arming pattern, read from shared memory so that the compiler
// treats them as sixteen live values (one consecutive block that every arming store re-uses)
// instead of re-creating sixteen constants in front of each store.
__device__ __forceinline__ void load_arm_block(uint32_t smem_addr, uint32_t* m) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(m[4 * i]), "=r"(m[4 * i + 1]), "=r"(m[4 * i + 2]), "=r"(m[4 * i + 3])
                 : "r"(smem_addr + 16 * i));
}

// CAUSAL: 0 rectangular / non-causal, 1 causal, 2 decided at run time (debug instantiations)
template <int D, int ALGO, bool K_PER_BLOCK, int CAUSAL, int DEBUG>
__global__ void __launch_bounds__(Cfg<D, ALGO>::THREADS, 1)
fused_attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const FusedParams prm) {
  using C = Cfg<D, ALGO>;
  constexpr int NSWG = C::NSWG;
  const bool causal = (CAUSAL == 2) ? (prm.causal != 0) : (CAUSAL == 1);
  constexpr bool DUMP = DEBUG == 1;      // copy out the first key tile's intermediates
  constexpr bool TIMELINE = DEBUG == 2;  // per-role clock stamps of one CTA
  // DEBUG == 3: the stalled-wait drill.  The producer leaves out the copy of one key tile (a
  // host-chosen index), so the wait for it can never be satisfied, and every wait gives up after
  // a tenth of a millisecond instead of most of a second: the whole unwind path runs (abort flag,
  // votes around the warp-synchronous instructions, drain of copies in flight, tensor-memory
  // release, status word) while the GPU and the context stay healthy.
  constexpr bool DRILL = DEBUG == 3;
  constexpr long long kLimit = DRILL ? 200000LL : kWaitCycleLimit;
  constexpr bool O_MAGIC = (ALGO == kPiper);  // the sage partial is FP32 and needs no conversion
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const Bars bars{smem_base + C::OFF_BAR};
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + C::OFF_MISC + 4);
  float* vec_ring = reinterpret_cast<float*>(smem + C::OFF_VEC);
  float2* stat_ring = reinterpret_cast<float2*>(smem + C::OFF_STAT);
  float* m_ring = reinterpret_cast<float*>(smem + C::OFF_MRING);

  // warpgroups: softmax 0, softmax 1, dequant, helpers (their order within the CTA makes no difference)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, wg = warp >> 2;
  const int bh = blockIdx.y;
  const int n_qt = prm.sq_pad / kQTile;
  const int qt = causal ? (n_qt - 1 - blockIdx.x) : blockIdx.x;  // causal: longest tiles first
  const int q0 = qt * kQTile;
  const int n_all = prm.sk_pad / kKeyTile;
  // key tiles of this CTA: all of them, those at or below the diagonal (causal), or one split's share
  const int t_begin = blockIdx.z * prm.tiles_per_split;
  const int n_tiles = causal ? min(n_all, 2 * qt + 2) : min(n_all - t_begin, prm.tiles_per_split);
  // DUMP instantiations (debug entry point only) copy the first key tile's intermediates out
  const bool dumping = DUMP && prm.dump != nullptr && bh == prm.dump_bh && qt == prm.dump_qt;
  const bool stamping = TIMELINE && prm.timeline != nullptr && bh == prm.dump_bh && qt == prm.dump_qt &&
                        ((tid & 127) == 0 || (lane == 0 && wg == NSWG + C::NDQ));

  // One thread per mbarrier (one thread initialising all of them costs a CTA most of a
  // microsecond before its first copy can be issued).
  if (tid < C::NUM_BARS) {
    constexpr int FIRST_S_FREE = 1 + 2 * NK + NV + NVEC, FIRST_PV_DONE = FIRST_S_FREE + NS + NP;
    constexpr int FIRST_O_EMPTY = FIRST_PV_DONE + NPV, FIRST_STAT = FIRST_O_EMPTY + NO;
    int count = 1;  // copies and products: one arrival (expect_tx / commit)
    if (tid >= FIRST_S_FREE && tid < FIRST_PV_DONE) count = 128;                 // s_free, p_ready: a softmax warpgroup
    else if (tid >= FIRST_O_EMPTY && tid < FIRST_STAT) count = 128 * C::NDQ;      // o_empty: the dequant threads
    else if (tid >= FIRST_STAT) count = 128;                                      // stat_full, m_ready
    mbar_init(bars.at(tid), count);
    fence_barrier_init();
  }
  if (tid == 0) *abort_flag = 0;
  if (tid < 16) reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MAGIC)[tid] = kMagicBits;
  constexpr int PROD_WARP = (NSWG + C::NDQ) * 4;
  constexpr int QK_WARP = PROD_WARP + 1;
  constexpr int PV_WARP = PROD_WARP + 2;
  if (warp == PROD_WARP) {
    if (lane == 0) { prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_v); }
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish();
    tc_fence_before();
  }
  // The kernel is launched chained to its predecessor in the stream (the prepass): everything up to
  // here touches only this CTA's shared and tensor memory; from here on the prepass's results are read.
  cudaGridDependencySynchronize();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The CTA starts with 128 (piper, 512 threads) or 168 (sage, 384 threads) registers per
  // thread; the dequant rows need more and the helper warpgroup far fewer, so each role
  // resizes its allocation on entry.
  if (wg == NSWG + C::NDQ) setmaxnreg_dec<C::REG_HELPER>();

#define HROLE_CONVERGED C::PRODUCER_CONVERGED
  if (warp == PROD_WARP && HLANE) {
    // ------------------------------------------------------------------ producer
    // All 32 lanes run the loop and the waits; the elected lane issues the copies.
    if (HELECT) {
      mbar_expect_tx(bars.q_full(), C::Q_BYTES);
      tma_load_2d(smem_base + C::OFF_Q, &tm_q, bars.q_full(), 0, bh * prm.sq_pad + q0);
      // A Q tile is read once, from DRAM, and nothing of its CTA can start before it has arrived:
      // the tile of the CTA about one wave further on (the one that will follow on some SM when
      // the current wave retires) is brought into L2 now.
      const long long next = static_cast<long long>(bh) * gridDim.x + blockIdx.x + kPrefetchCtasAhead;
      if (blockIdx.z == 0 && next < static_cast<long long>(gridDim.x) * gridDim.y) {
        const int nbh = static_cast<int>(next / gridDim.x), nx = static_cast<int>(next % gridDim.x);
        const int nqt = causal ? (n_qt - 1 - nx) : nx;
        tma_prefetch_l2_2d(&tm_q, 0, nbh * prm.sq_pad + nqt * kQTile);
      }
    }
    const long long vec_base = static_cast<long long>(bh) * prm.sk_pad;
    int last = -1;  // last key tile whose copies were issued
    // The producer runs a whole ring ahead of the products, so its waits have microseconds of
    // slack: the piper producer sleeps between probes instead of taking issue slots from the
    // compute warps of its scheduler (1.5 % at long key sequences; nothing for sage).
    auto producer_wait = [&](uint32_t bar, uint32_t parity, int where) -> bool {
      if (C::PRODUCER_SLEEP_NS > 0) return mbar_wait_relaxed<(C::PRODUCER_SLEEP_NS > 0 ? C::PRODUCER_SLEEP_NS : 1)>(bar, parity, abort_flag, where, kLimit);
      return mbar_wait_bounded(bar, parity, abort_flag, where, kLimit);
    };
    for (int i = 0; i < n_tiles; ++i) {
      PK_STAMP(NSWG + 3, i, 0);
      const int ks = i % NK, vs = i % NV, cs = i % NVEC;
      // K stage ks was last read by S_{i-NK}, V stage vs by PV_{i-NV}.  The vector slot of tile
      // i-NVEC was last read before the probabilities of that tile were published, which
      // precedes the completion of S_{i-NK} (NVEC >= NK + NS + 2).
      if (i >= NK && !HWAIT(producer_wait(bars.qk_done(ks), ((i / NK) - 1) & 1, W_PROD_K))) break;
      PK_STAMP(NSWG + 3, i, 1);
      if (i >= NV && !HWAIT(producer_wait(bars.pv_done(i % NPV), ((i / NPV) - 1) & 1, W_PROD_V))) break;
      if (HELECT) {
        if (!(DRILL && i == prm.skip_key_tile)) {
          mbar_expect_tx(bars.k_full(ks), C::K_BYTES);
          tma_load_2d(smem_base + C::OFF_K + ks * C::K_BYTES, &tm_k, bars.k_full(ks), 0, bh * prm.sk_pad + (t_begin + i) * kKeyTile);
        }
        const uint32_t vdst = smem_base + C::OFF_VEC + cs * VEC_FLOATS * 4;
        const uint32_t vbar = bars.vec_full(cs);
        mbar_expect_tx(vbar, VEC_FLOATS * 4);
        const long long off = vec_base + static_cast<long long>(t_begin + i) * kKeyTile;
        bulk_load(vdst, prm.k_mul + off, kKeyTile * 4, vbar);
        bulk_load(vdst + kKeyTile * 4, prm.k_add + off, kKeyTile * 4, vbar);
        bulk_load(vdst + 2 * kKeyTile * 4, prm.k_inv + off, kKeyTile * 4, vbar);
        mbar_expect_tx(bars.v_full(vs), C::V_BYTES);
        tma_load_2d(smem_base + C::OFF_V + vs * C::V_BYTES, &tm_v, bars.v_full(vs), (t_begin + i) * kKeyTile, bh * D);
      }
      last = i;
      PK_STAMP(NSWG + 3, i, 2);
    }
    if (*abort_flag != 0) {
      // Giving up: let the copies this warp has issued land (each wait is short and raises nothing)
      // before the CTA returns and its shared memory is handed to another CTA.
      constexpr long long kDrain = 100000;
      mbar_wait_quiet(bars.q_full(), 0, kDrain);
      for (int t = max(0, last - NK + 1); t <= last; ++t) {
        if (!(DRILL && t == prm.skip_key_tile)) mbar_wait_quiet(bars.k_full(t % NK), (t / NK) & 1, kDrain);
      }
      for (int t = max(0, last - NVEC + 1); t <= last; ++t) mbar_wait_quiet(bars.vec_full(t % NVEC), (t / NVEC) & 1, kDrain);
      for (int t = max(0, last - NV + 1); t <= last; ++t) mbar_wait_quiet(bars.v_full(t % NV), (t / NV) & 1, kDrain);
    }
#undef HROLE_CONVERGED
#define HROLE_CONVERGED true
  } else if (warp == QK_WARP && HLANE) {
    // ------------------------------------------------------------------ S = Q K^T issue
    // The two products are issued by two different warps.  S_j is issued as soon as K tile j has
    // landed and score buffer j % NS has been read and re-armed by the softmax warpgroup.
    constexpr uint32_t idesc_qk = umma_idesc(kAccS32, kFmtS8, kFmtS8, kQTile, kKeyTile);
    const uint64_t qdesc = umma_smem_desc(smem_base + C::OFF_Q, D);
    const uint64_t kdesc0 = umma_smem_desc(smem_base + C::OFF_K, D);
    bool ok = HWAIT(mbar_wait_bounded(bars.q_full(), 0, abort_flag, W_QK_Q, kLimit));
    for (int j = 0; ok && j < n_tiles; ++j) {
      PK_STAMP(NSWG + 1, j, 0);
      if (!HWAIT(mbar_wait_bounded(bars.k_full(j % NK), (j / NK) & 1, abort_flag, W_QK_K, kLimit))) break;
      if (!HWAIT(mbar_wait_bounded(bars.s_free(j % NS), (j / NS) & 1, abort_flag, W_QK_S, kLimit))) break;
      tc_fence_after();
      PK_STAMP(NSWG + 1, j, 1);
      const uint64_t kdesc = kdesc0 + static_cast<uint64_t>(((j % NK) * C::K_BYTES) >> 4);
      const uint32_t d = tmem_base + C::COL_S + (j % NS) * kKeyTile;
      if (HELECT) {
#pragma unroll
        for (int kk = 0; kk < D / 32; ++kk) umma_i8_ss(d, qdesc + 2 * kk, kdesc + 2 * kk, idesc_qk, 1u);
        tc_commit(bars.qk_done(j % NK));
      }
      PK_STAMP(NSWG + 1, j, 2);
    }
  } else if (warp == PV_WARP && HLANE) {
    // ------------------------------------------------------------------ O_part = P V issue
    constexpr uint32_t idesc_pv = (ALGO == kPiper) ? umma_idesc(kAccS32, kFmtU8, kFmtS8, kQTile, D)
                                                   : umma_idesc(kAccF32, kFmtE4M3, kFmtE4M3, kQTile, D);
    const uint64_t vdesc0 = umma_smem_desc(smem_base + C::OFF_V, kKeyTile);
    for (int j = 0; j < n_tiles; ++j) {
      PK_STAMP(NSWG + 2, j, 0);
      if (!HWAIT(mbar_wait_bounded(bars.p_ready(j % NP), (j / NP) & 1, abort_flag, W_PV_P, kLimit))) break;
      if (!HWAIT(mbar_wait_bounded(bars.o_empty(j % NO), (j / NO) & 1, abort_flag, W_PV_O, kLimit))) break;
      if (!HWAIT(mbar_wait_bounded(bars.v_full(j % NV), (j / NV) & 1, abort_flag, W_PV_V, kLimit))) break;
      tc_fence_after();
      PK_STAMP(NSWG + 2, j, 1);
      const uint64_t vdesc = vdesc0 + static_cast<uint64_t>(((j % NV) * C::V_BYTES) >> 4);
      const uint32_t d = tmem_base + C::COL_O + (j % NO) * D;
      const uint32_t a = tmem_base + C::COL_P + (j % NP) * (kKeyTile / 4);
      if (HELECT) {
#pragma unroll
        for (int kk = 0; kk < kKeyTile / 32; ++kk) {
          if (ALGO == kPiper) umma_i8_ts(d, a + 8 * kk, vdesc + 2 * kk, idesc_pv, 1u);
          else umma_f8_ts(d, a + 8 * kk, vdesc + 2 * kk, idesc_pv, kk > 0);
        }
        tc_commit(bars.pv_done(j % NPV));
      }
      PK_STAMP(NSWG + 2, j, 2);
    }
#undef HROLE_CONVERGED
  } else if (wg == NSWG + C::NDQ) {
    // idle lanes / the fourth helper warp
  } else if (wg < NSWG) {
    // ------------------------------------------------------------------ softmax
    if (C::REG_SM <= C::LAUNCH_REGS) setmaxnreg_dec<C::REG_SM>(); else setmaxnreg_inc<C::REG_SM>();
    const int row = tid & 127;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const float qm = prm.q_mul[static_cast<long long>(bh) * prm.sq_pad + q0 + row];
    float m_run = -INFINITY;  // sage only
    if (wg == 0) {  // arm every score buffer, then hand them to the mma warp
      tmem_arm(lane_addr + C::COL_S, NS * kKeyTile);
      tmem_wait_st();
      tc_fence_before();
      for (int i = 0; i < NS; ++i) mbar_arrive(bars.s_free(i));
    }
    const float2 neg_magic2 = make_float2(-kMagic, -kMagic);
    uint32_t armv[16];
    load_arm_block(smem_base + C::OFF_MAGIC, armv);
    // Sage with per-key K scales: t_c = q_mul * (score_c * k_mul_c), nothing added but -inf on
    // padding, so the row factor can wait until the shift in front of the exponential.
    constexpr bool ROW_SCALE_LATE = ALGO == kSage && !K_PER_BLOCK;
    for (int j = wg; j < n_tiles; j += NSWG) {
      PK_STAMP(wg, j, 0);
      // votes keep the warp converged for the .sync.aligned tensor-memory ops even when a wait is abandoned
      if (!WARP_ALL(mbar_wait_bounded(bars.vec_full(j % NVEC), (j / NVEC) & 1, abort_flag, W_SM_VEC, kLimit))) break;
      if (!WARP_ALL(mbar_wait_bounded(bars.qk_done(j % NK), (j / NK) & 1, abort_flag, W_SM_S, kLimit))) break;
      tc_fence_after();
      PK_STAMP(wg, j, 1);
      const uint32_t s_addr = lane_addr + C::COL_S + (j % NS) * kKeyTile;
      // Per-key vectors of this tile in shared memory: [0,64) K scale, [64,128) additive term
      // (log2 of the V row scale / 0, -inf on padding), [128,192) 1 / V row scale.
      const float4* vk = reinterpret_cast<const float4*>(vec_ring + (j % NVEC) * VEC_FLOATS);
      const float mt = K_PER_BLOCK ? qm * vec_ring[(j % NVEC) * VEC_FLOATS] : qm;
      const float2 mt2 = make_float2(mt, mt);
      const bool diag = causal && (j * kKeyTile + kKeyTile - 1 > q0);
      const int lim = q0 + row - j * kKeyTile;  // causal: columns above this index are masked

      // t_c = score_c * (q_mul * k_mul_c) + k_add_c for the 16 columns of chunk `ch`, two columns
      // per packed FP32 instruction; the word read from tensor memory is the float 1.5*2^23 + score.
      auto scores16 = [&](const uint32_t* sr, int ch, float2* t2) {
        if (DUMP) {
          if (dumping && j == 0) {
            int32_t* ds = static_cast<int32_t*>(prm.dump);
#pragma unroll
            for (int c = 0; c < 16; ++c) ds[row * kKeyTile + ch * 16 + c] = static_cast<int32_t>(sr[c] - kMagicBits);
          }
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const float4 add = vk[kKeyTile / 4 + ch * 4 + q4];
          const float2 f0 = __fadd2_rn(make_float2(__uint_as_float(sr[q4 * 4 + 0]), __uint_as_float(sr[q4 * 4 + 1])), neg_magic2);
          const float2 f1 = __fadd2_rn(make_float2(__uint_as_float(sr[q4 * 4 + 2]), __uint_as_float(sr[q4 * 4 + 3])), neg_magic2);
          if (K_PER_BLOCK) {
            t2[q4 * 2 + 0] = __ffma2_rn(f0, mt2, make_float2(add.x, add.y));
            t2[q4 * 2 + 1] = __ffma2_rn(f1, mt2, make_float2(add.z, add.w));
          } else if (ROW_SCALE_LATE) {
            // u_c = score_c * k_mul_c (+ -inf on padding); the positive row factor q_mul is applied
            // with the shift in front of the exponential, one multiplication per pair fewer
            const float4 mul = vk[ch * 4 + q4];
            t2[q4 * 2 + 0] = __ffma2_rn(f0, make_float2(mul.x, mul.y), make_float2(add.x, add.y));
            t2[q4 * 2 + 1] = __ffma2_rn(f1, make_float2(mul.z, mul.w), make_float2(add.z, add.w));
          } else {
            const float4 mul = vk[ch * 4 + q4];
            t2[q4 * 2 + 0] = __ffma2_rn(__fmul2_rn(f0, mt2), make_float2(mul.x, mul.y), make_float2(add.x, add.y));
            t2[q4 * 2 + 1] = __ffma2_rn(__fmul2_rn(f1, mt2), make_float2(mul.z, mul.w), make_float2(add.z, add.w));
          }
        }
        if (diag) {
#pragma unroll
          for (int c2 = 0; c2 < 8; ++c2) {
            if (ch * 16 + 2 * c2 > lim) t2[c2].x = -INFINITY;
            if (ch * 16 + 2 * c2 + 1 > lim) t2[c2].y = -INFINITY;
          }
        }
      };

      // Single pass over registers: the whole 64-column tile is loaded once, the score buffer is
      // re-armed at once (and handed back after the exponentials), and t stays in registers between
      // max and exp.
      uint32_t sraw[kKeyTile];
      tmem_ld32(s_addr, sraw);
      tmem_ld32(s_addr + 32, sraw + 32);
      tmem_wait_ld();
      PK_STAMP(wg, j, 4);
#pragma unroll
      for (int c16 = 0; c16 < kKeyTile; c16 += 16) tmem_st16(s_addr + c16, armv);
      float2 t2[kKeyTile / 2];
#pragma unroll
      for (int ch = 0; ch < kKeyTile / 16; ++ch) scores16(sraw + ch * 16, ch, t2 + ch * 8);
      float bm0 = fmaxf(t2[0].x, t2[0].y), bm1 = fmaxf(t2[1].x, t2[1].y);
#pragma unroll
      for (int c2 = 2; c2 < kKeyTile / 2; c2 += 2) { bm0 = max3(bm0, t2[c2].x, t2[c2].y); bm1 = max3(bm1, t2[c2 + 1].x, t2[c2 + 1].y); }
      // ROW_SCALE_LATE: the maximum was taken over u; q_mul > 0 commutes with it
      const float bm = ROW_SCALE_LATE ? fmaxf(bm0, bm1) * mt : fmaxf(bm0, bm1);
      PK_STAMP(wg, j, 2);
      float shift, ow = 1.f;
      if (ALGO == kPiper) {
        shift = (bm == -INFINITY) ? 0.f : -bm;
      } else {
        // Sage's codes are relative to the running maximum.  With two softmax warpgroups on
        // alternate tiles the maximum after tile j-1 comes from the other warpgroup through shared
        // memory; only this short hand-over is sequential, the exponentials of consecutive tiles
        // overlap.
        if (NSWG > 1 && j > 0) {
          if (!WARP_ALL(mbar_wait_bounded(bars.m_ready((j - 1) % NM), ((j - 1) / NM) & 1, abort_flag, W_SM_M, kLimit))) break;
          m_run = m_ring[((j - 1) % NM) * kQTile + row];
        }
        const float nm = fmaxf(m_run, bm);
        if (NSWG > 1) {
          m_ring[(j % NM) * kQTile + row] = nm;
          mbar_arrive(bars.m_ready(j % NM));
        }
        const float ns = (nm == -INFINITY) ? 0.f : nm;
        ow = (m_run == nm) ? 1.f : ex2_approx(m_run - ns);
        shift = 8.807354922057604f - ns;  // log2(448): P = e4m3(448 * 2^(t - max))
        m_run = nm;
      }
      const float2 shift2 = make_float2(shift, shift);
      const float2 c255 = make_float2(255.f, 255.f), magic2 = make_float2(kMagic, kMagic);
      float2 psum_a = make_float2(0.f, 0.f), psum_b = make_float2(0.f, 0.f);
      uint32_t packed[kKeyTile / 4];
#pragma unroll
      for (int c4 = 0; c4 < kKeyTile / 4; ++c4) {
        const float2 d0 = ROW_SCALE_LATE ? __ffma2_rn(t2[c4 * 2 + 0], mt2, shift2) : __fadd2_rn(t2[c4 * 2 + 0], shift2);
        const float2 d1 = ROW_SCALE_LATE ? __ffma2_rn(t2[c4 * 2 + 1], mt2, shift2) : __fadd2_rn(t2[c4 * 2 + 1], shift2);
        const float2 e0 = make_float2(ex2_approx(d0.x), ex2_approx(d0.y));
        const float2 e1 = make_float2(ex2_approx(d1.x), ex2_approx(d1.y));
        if (ALGO == kPiper) {
          const float4 inv = vk[2 * (kKeyTile / 4) + c4];
          psum_a = __ffma2_rn(e0, make_float2(inv.x, inv.y), psum_a);
          psum_b = __ffma2_rn(e1, make_float2(inv.z, inv.w), psum_b);
          const float2 b0 = __ffma2_rn(e0, c255, magic2), b1 = __ffma2_rn(e1, c255, magic2);  // low byte = rne(255 e)
          const uint32_t lo = __byte_perm(__float_as_uint(b0.x), __float_as_uint(b0.y), 0x0040);
          const uint32_t hi = __byte_perm(__float_as_uint(b1.x), __float_as_uint(b1.y), 0x0040);
          packed[c4] = __byte_perm(lo, hi, 0x5410);
        } else {
          psum_a = __fadd2_rn(psum_a, e0);
          psum_b = __fadd2_rn(psum_b, e1);
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(e0, __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(e1, __NV_SATFINITE, __NV_E4M3);
          packed[c4] = __byte_perm(lo, hi, 0x5410);
        }
      }
      PK_STAMP(wg, j, 5);
      // The score buffer goes back to the S issue warp only now (its arming stores have long
      // landed, so the wait costs nothing; the S products run two tiles ahead anyway): handing it
      // back right after the maximum put a tensor-memory wait into the middle of the arithmetic.
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bars.s_free(j % NS));
      // probability buffer j%NP was last read by the PV product of tile j-NP
      if (j >= NP && !WARP_ALL(mbar_wait_bounded(bars.pv_done((j - NP) % NPV), ((j - NP) / NPV) & 1, abort_flag, W_SM_PV, kLimit))) break;
      tc_fence_after();
      PK_STAMP(wg, j, 6);
      const uint32_t p_addr = lane_addr + C::COL_P + (j % NP) * (kKeyTile / 4);
      tmem_st16(p_addr, packed);
      if (DUMP) {
        if (dumping && j == 0) {
          uint32_t* dp = reinterpret_cast<uint32_t*>(static_cast<char*>(prm.dump) + kQTile * kKeyTile * 4);
#pragma unroll
          for (int c = 0; c < kKeyTile / 4; ++c) dp[row * (kKeyTile / 4) + c] = packed[c];
        }
      }
      const float psum = (psum_a.x + psum_a.y) + (psum_b.x + psum_b.y);
      const float2 st = (ALGO == kPiper) ? make_float2(bm, psum) : make_float2(ow, psum * (1.f / 448.f));
      stat_ring[(j % NSTAT) * kQTile + row] = st;
      tmem_wait_st();
      PK_STAMP(wg, j, 7);
      tc_fence_before();
      mbar_arrive(bars.p_ready(j % NP));
      mbar_arrive(bars.stat_full(j % NSTAT));
      PK_STAMP(wg, j, 3);
    }
  } else if (wg < NSWG + C::NDQ) {
    // ------------------------------------------------------------------ dequant + epilogue
    setmaxnreg_inc<C::REG_DQ>();
    constexpr int DH = D / C::NDQ;          // columns folded by this warpgroup
    constexpr int CH = 16;                  // columns per tensor-memory round trip
    const int col0 = (wg - NSWG) * DH;      // first of them
    const int row = tid & 127;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    if (O_MAGIC) {
      for (int i = 0; i < NO; ++i) tmem_arm(lane_addr + C::COL_O + i * D + col0, DH);
      tmem_wait_st();
    }
    tc_fence_before();
    for (int i = 0; i < NO; ++i) mbar_arrive(bars.o_empty(i));

    // The epilogue adds the V mean (multiplies by the V scale) of every column: fetched now, one
    // float per thread, so that its trip to L2 is over long before the values are needed.
    float* aux_s = reinterpret_cast<float*>(smem + C::OFF_AUX);
    if (row < D) aux_s[row] = prm.v_aux[static_cast<long long>(bh) * D + row];

    float2 num2[DH / 2];
#pragma unroll
    for (int d = 0; d < DH / 2; ++d) num2[d] = make_float2(0.f, 0.f);
    float den = 0.f, m = -INFINITY;
    bool ok = true;
    // Row statistics recurrence (running max, denominator, rescale factors).  It depends only on
    // the per-tile statistics that the softmax warpgroups publish several tiles ahead, so the
    // factors of tile j+1 are evaluated early in the fold of tile j, where the chain of dependent
    // instructions (shared-memory load, an exponential) overlaps the fold arithmetic.
    constexpr float kRescaleThreshold = 8.f;
    float ow = 1.f, c = 0.f;      // factors of the tile being folded
    float ow_n = 1.f, c_n = 0.f;  // factors of the next tile
    auto advance_stats = [&](int j) -> bool {
      if (!WARP_ALL(mbar_wait_bounded(bars.stat_full(j % NSTAT), (j / NSTAT) & 1, abort_flag, W_DQ_STAT, kLimit))) return false;
      const float2 st = stat_ring[(j % NSTAT) * kQTile + row];
      if (ALGO == kPiper) {
        const float bm = st.x;
        // `m` is the exponent the numerators and the denominator are relative to.  It follows the
        // tiles' maxima lazily: only a tile whose maximum exceeds it by more than
        // kRescaleThreshold moves it (and costs a pass over the numerator row); otherwise the
        // tile's weight 2^(bm - m) simply exceeds one, by at most 2^kRescaleThreshold.  num / den
        // is the same quotient for any reference exponent; only FP32 rounding differs (1e-7).
        float cw;
        if (bm == -INFINITY) { ow_n = 1.f; cw = 0.f; }
        else if (bm > m + kRescaleThreshold) { ow_n = ex2_approx(m - bm); cw = 1.f; m = bm; }
        else { ow_n = 1.f; cw = ex2_approx(bm - m); }
        den = fmaf(den, ow_n, st.y * cw);
        c_n = cw * (1.f / 255.f);
      } else {
        ow_n = st.x;
        den = fmaf(den, ow_n, st.y);
        c_n = 1.f;
      }
      return true;
    };
    // The partial is read CH columns at a time; the next chunk's load is in flight while the
    // current one is folded, and each chunk is re-armed once read.  FOLD_FROM_TILE_TOP: the
    // tile's factors are evaluated and its product awaited before its first chunk is requested.
    // Otherwise both happen one tile ahead (at chunk STAT_AT / NEXT_AT of the previous tile) and
    // the first chunk of tile j+1 is requested before the last chunk of tile j is folded.
    constexpr int NCH = DH / CH;
    static_assert(NCH >= 2, "the next tile's product is waited for before the last chunk");
    constexpr int STAT_AT = 1;  // chunk after which the next tile's factors are evaluated
    // ... and the next tile's product awaited.  Which chunk makes no difference as long as the two
    // stay together: every wait splits the unrolled fold into another block (6-7 % per split).
    constexpr int NEXT_AT = 1;
    uint32_t obuf[2][CH];
    const float2 neg_magic2 = make_float2(-kMagic, -kMagic);
    uint32_t armv[16];
    load_arm_block(smem_base + C::OFF_MAGIC, armv);
    if (!C::FOLD_FROM_TILE_TOP && n_tiles > 0) {
      ok = advance_stats(0);
      ok = ok && WARP_ALL(mbar_wait_bounded(bars.pv_done(0), 0, abort_flag, W_DQ_O, kLimit));
      if (ok) {
        tc_fence_after();
        tmem_ldN<CH>(lane_addr + C::COL_O + col0, obuf[0]);
      }
    }
    for (int j = 0; ok && j < n_tiles; ++j) {
      PK_STAMP(NSWG, j, 0);
      const uint32_t o_addr = lane_addr + C::COL_O + (j % NO) * D + col0;
      if (C::FOLD_FROM_TILE_TOP) {
        ok = advance_stats(j);
        PK_STAMP(NSWG, j, 7);
        ok = ok && WARP_ALL(mbar_wait_bounded(bars.pv_done(j % NPV), (j / NPV) & 1, abort_flag, W_DQ_O, kLimit));
        if (!ok) break;
        tc_fence_after();
        PK_STAMP(NSWG, j, 5);
        tmem_ldN<CH>(o_addr, obuf[0]);
      }
      ow = ow_n; c = c_n;
      if (WARP_ANY(ow != 1.f)) {
        const float2 ow2 = make_float2(ow, ow);
#pragma unroll
        for (int d = 0; d < DH / 2; ++d) num2[d] = __fmul2_rn(num2[d], ow2);
      }
      const float2 c2 = make_float2(c, c);
      PK_STAMP(NSWG, j, 1);
#pragma unroll
      for (int ch = 0; ch < NCH; ++ch) {
        tmem_wait_ld();
        if (ch == 0) PK_STAMP(NSWG, j, 2);
        if (ch + 1 < NCH) {
          tmem_ldN<CH>(o_addr + (ch + 1) * CH, obuf[(ch + 1) & 1]);
        } else if (!C::FOLD_FROM_TILE_TOP && j + 1 < n_tiles && ok) {
          // first chunk of the next tile (its product was waited for below, chunks ago)
          tmem_ldN<CH>(lane_addr + C::COL_O + ((j + 1) % NO) * D + col0, obuf[(ch + 1) & 1]);
        }
        if (!C::FOLD_FROM_TILE_TOP && ch == STAT_AT && j + 1 < n_tiles) {
          PK_STAMP(NSWG, j, 4);
          ok = advance_stats(j + 1);
          PK_STAMP(NSWG, j, 7);
        }
        if (!C::FOLD_FROM_TILE_TOP && ch == NEXT_AT && j + 1 < n_tiles) {
          ok = ok && WARP_ALL(mbar_wait_bounded(bars.pv_done((j + 1) % NPV), ((j + 1) / NPV) & 1, abort_flag, W_DQ_O, kLimit));
          tc_fence_after();
          PK_STAMP(NSWG, j, 5);
        }
        if (O_MAGIC) {
#pragma unroll
          for (int c16 = 0; c16 < CH; c16 += 16) tmem_st16(o_addr + ch * CH + c16, armv);
        }
        const uint32_t* o = obuf[ch & 1];
        if (DUMP && dumping && j == 0) {
          uint32_t* dp = reinterpret_cast<uint32_t*>(static_cast<char*>(prm.dump) + kQTile * kKeyTile * 5);
#pragma unroll
          for (int i = 0; i < CH; ++i) dp[row * D + col0 + ch * CH + i] = O_MAGIC ? o[i] - kMagicBits : o[i];
        }
#pragma unroll
        for (int i = 0; i < CH / 2; ++i) {
          float2 y = make_float2(__uint_as_float(o[2 * i]), __uint_as_float(o[2 * i + 1]));
          if (ALGO == kPiper) {
            // the word is the float 1.5*2^23 + partial; num += partial * c
            num2[ch * (CH / 2) + i] = __ffma2_rn(__fadd2_rn(y, neg_magic2), c2, num2[ch * (CH / 2) + i]);
          } else {
            num2[ch * (CH / 2) + i] = __fadd2_rn(num2[ch * (CH / 2) + i], __half22float2(__floats2half2_rn(y.x, y.y)));
          }
        }
      }
      PK_STAMP(NSWG, j, 6);
      if (O_MAGIC) tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bars.o_empty(j % NO));
      PK_STAMP(NSWG, j, 3);
    }
    // epilogue: normalise, restore the V mean (piper) / apply the channel scale (sage), cast
    const int grow = q0 + row;
    if (!ok && grow < prm.Sq && prm.splits == 1) {
      // A wait was abandoned: this tile's rows are not valid.  They are filled with NaN so that a
      // caller who never reads the status words cannot mistake them for results.
      const long long obase = (static_cast<long long>(bh) * prm.Sq + grow) * D + col0;
      for (int d0 = 0; d0 < DH; ++d0) {
        if (prm.out_dtype == PK_F32) static_cast<float*>(prm.out)[obase + d0] = __int_as_float(0x7FC00000);
        else static_cast<uint16_t*>(prm.out)[obase + d0] = (prm.out_dtype == PK_F16) ? 0x7E00 : 0x7FC0;
      }
    }
    if (prm.splits > 1) {
      // Key-split launch: leave the un-normalised row (numerators relative to 2^max, the running
      // maximum and the denominator) for the merge kernel.  Padding rows are written too (zeros).
      float mx = m;  // piper: tracked here; sage: the softmax warpgroups' last hand-over value
      if (ALGO == kSage) mx = n_tiles > 0 ? m_ring[((n_tiles - 1) % NM) * kQTile + row] : -INFINITY;
      float* pr = prm.partial + ((static_cast<long long>(bh) * prm.sq_pad + q0 + row) * prm.splits + blockIdx.z) * (D + 4) + col0;
      const float bad = __int_as_float(0x7FC00000);
#pragma unroll
      for (int d0 = 0; d0 < DH; d0 += 4)
        *reinterpret_cast<float4*>(pr + d0) = make_float4(num2[d0 / 2].x, num2[d0 / 2].y, num2[d0 / 2 + 1].x, num2[d0 / 2 + 1].y);
      *reinterpret_cast<float4*>(pr + DH) = make_float4(mx, ok ? den : bad, 0.f, 0.f);
    } else {
      // Each thread holds one output row.  Stored from here, a warp's store instruction would touch
      // 32 rows with 16 bytes each (that epilogue took 6 us per CTA, 11 % of a 64-key-tile CTA).
      // The rows go through shared memory instead (the K/V rings are idle by now: every product
      // has completed), padded by 16 bytes so that the 8 lanes of a store phase hit different
      // banks, and leave as whole rows: 32 lanes x 16 bytes of consecutive addresses.
      static_assert(C::NDQ == 1, "the staging area is laid out for one dequant warpgroup");
      static_assert(4 * 32 * (D * 4 + 16) <= NK * C::K_BYTES + NV * C::V_BYTES, "staging fits into the K/V rings");
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the dequant warpgroup's aux_s writes, made before its main loop
      const int esz = (prm.out_dtype == PK_F32) ? 4 : 2;
      const int row_bytes = D * esz, stride = row_bytes + 16;
      uint8_t* stage = smem + C::OFF_K + (warp & 3) * 32 * (D * 4 + 16);
      if (ok && grow < prm.Sq) {
        // one IEEE division per row; the D per-element divisions of the reference become
        // multiplications by the reciprocal (at most an ulp apart, and far less code)
        const float dinv = __fdiv_rn(1.f, fmaxf(den, 1e-30f));
        const float4* aux4 = reinterpret_cast<const float4*>(aux_s);
        uint8_t* mine = stage + lane * stride;
#pragma unroll
        for (int d0 = 0; d0 < D; d0 += 8) {
          const float4 a0 = aux4[d0 / 4], a1 = aux4[d0 / 4 + 1];
          const float aux[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          float r[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float nv = (i & 1) ? num2[(d0 + i) / 2].y : num2[(d0 + i) / 2].x;
            if (ALGO == kPiper) r[i] = fmaf(nv, dinv, aux[i]);
            else r[i] = nv * (aux[i] * (1.f / 448.f)) * dinv;
          }
          if (prm.out_dtype == PK_F32) {
            float4* o = reinterpret_cast<float4*>(mine + d0 * 4);
            o[0] = make_float4(r[0], r[1], r[2], r[3]);
            o[1] = make_float4(r[4], r[5], r[6], r[7]);
          } else {
            uint32_t pk4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (prm.out_dtype == PK_F16) {
                const __half2 h = __floats2half2_rn(r[2 * i], r[2 * i + 1]);
                pk4[i] = *reinterpret_cast<const uint32_t*>(&h);
              } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * i], r[2 * i + 1]);
                pk4[i] = *reinterpret_cast<const uint32_t*>(&h);
              }
            }
            *reinterpret_cast<uint4*>(mine + d0 * 2) = make_uint4(pk4[0], pk4[1], pk4[2], pk4[3]);
          }
        }
      }
      __syncwarp();
      if (ok) {  // uniform within the warp (every wait result is voted on)
        const int lanes_per_row = row_bytes / 16, rows_per_store = 32 / lanes_per_row;
        const int sub = lane / lanes_per_row, piece = lane % lanes_per_row;
        const int first_row = q0 + (warp & 3) * 32;
        uint8_t* out_bytes = static_cast<uint8_t*>(prm.out);
        for (int it = 0; it < 32 / rows_per_store; ++it) {
          const int rl = it * rows_per_store + sub;
          if (first_row + rl < prm.Sq) {
            const uint4 val = *reinterpret_cast<const uint4*>(stage + rl * stride + piece * 16);
            *reinterpret_cast<uint4*>(out_bytes + (static_cast<long long>(bh) * prm.Sq + first_row + rl) * row_bytes + piece * 16) = val;
          }
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
  if (tid == 0 && *abort_flag != 0) {
    atomicCAS(prm.status, 0, *abort_flag);
    if (prm.host_status != nullptr) atomicCAS_system(prm.host_status, 0, *abort_flag);
  }
}

// ---------------------------------------------------------------------------------------
// Merge of a key-split launch: one warp per query row combines the splits' un-normalised rows,
// out = sum_s num_s 2^(m_s - M) / sum_s den_s 2^(m_s - M), then the usual epilogue.
// ---------------------------------------------------------------------------------------
template <int D, int ALGO>
__global__ void __launch_bounds__(256) merge_splits_kernel(const float* __restrict__ partial, const float* __restrict__ v_aux,
                                                           void* __restrict__ out, int out_dtype, int Sq, int sq_pad,
                                                           int splits, long long rows_total) {
  constexpr int VEC = D / 32;  // columns per lane
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  // Launched with programmatic stream serialisation: this kernel may start while the fused kernel
  // is still running (its launch latency hides behind that kernel's tail); the partial rows are
  // complete and visible once this returns.
  cudaGridDependencySynchronize();
  if (gw >= rows_total) return;
  const long long bh = gw / Sq;
  const int row = static_cast<int>(gw % Sq);
  const float* pr = partial + ((bh * sq_pad + row) * splits) * (D + 4);
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, pr[s * (D + 4) + D]);
  float den = 0.f, acc[VEC];
  bool bad = false;
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float* ps = pr + s * (D + 4);
    const float ms = ps[D], ds = ps[D + 1];
    bad |= ds != ds;  // a split that gave up a wait marks its denominator
    const float w = (ms == mx) ? 1.f : ex2_approx(ms - mx);
    den = fmaf(ds, w, den);
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = fmaf(ps[lane * VEC + i], w, acc[i]);
  }
  const float dinv = bad ? __int_as_float(0x7FC00000) : __fdiv_rn(1.f, fmaxf(den, 1e-30f));
  const float* aux = v_aux + bh * D + lane * VEC;
  const long long obase = (bh * Sq + row) * D + lane * VEC;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const float r = (ALGO == kPiper) ? fmaf(acc[i], dinv, aux[i]) : acc[i] * (aux[i] * (1.f / 448.f)) * dinv;
    if (out_dtype == PK_F32) static_cast<float*>(out)[obase + i] = r;
    else if (out_dtype == PK_F16) static_cast<__half*>(out)[obase + i] = __float2half_rn(r);
    else static_cast<__nv_bfloat16*>(out)[obase + i] = __float2bfloat16_rn(r);
  }
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

template <int D, int ALGO, bool KPB, int CAUSAL, int DEBUG>
int launch_one_impl(const pk_problem& p, const Layout& L, cudaStream_t st, const DebugDump* dump) {
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
  prm.timeline = dump ? static_cast<long long*>(dump->timeline) : nullptr;
  prm.timeline_tiles = dump ? dump->timeline_tiles : 0;
  prm.skip_key_tile = dump ? dump->skip_key_tile : -1;
  prm.host_status = fault_word_device_ptr(p.device);
  // the debug instantiations always run unsplit
  const int splits = (DEBUG == 0) ? L.splits : 1;
  prm.splits = splits;
  prm.tiles_per_split = splits > 1 ? L.tiles_per_split : L.sk_pad / kKeyTile;
  prm.partial = splits > 1 ? at<float>(p, L.partial) : nullptr;
  auto kern = fused_attention_kernel<D, ALGO, KPB, CAUSAL, DEBUG>;
  {
    // the attribute is per function and device: set it once
    static std::atomic<bool> done[64];
    const int dev = (p.device >= 0 && p.device < 64) ? p.device : 0;
    if (!done[dev].load(std::memory_order_acquire)) {
      const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
      if (e != cudaSuccess) return fail(PK_ERR_CUDA, "cudaFuncSetAttribute: %s", cuda_err(e));
      done[dev].store(true, std::memory_order_release);
    }
  }
  const dim3 grid(L.sq_pad / kQTile, L.BH, splits);
  cudaError_t e = launch_chained(kern, grid, dim3(C::THREADS), C::SMEM_BYTES, st, tq, tk, tv, prm);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PK_ERR_CUDA, "fused kernel launch failed: %s", cuda_err(e));
  if (splits > 1) {
    const long long rows = static_cast<long long>(L.BH) * L.Sq;
    const unsigned blocks = static_cast<unsigned>((rows * 32 + 255) / 256);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const float* partial_c = prm.partial;
    const float* aux_c = prm.v_aux;
    void* out_c = p.out;
    int out_dtype_c = p.out_dtype, sq_c = L.Sq, sq_pad_c = L.sq_pad, splits_c = splits;
    long long rows_c = rows;
    e = cudaLaunchKernelEx(&cfg, merge_splits_kernel<D, ALGO>, partial_c, aux_c, out_c, out_dtype_c, sq_c, sq_pad_c, splits_c, rows_c);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(PK_ERR_CUDA, "merge kernel launch failed: %s", cuda_err(e));
  }
  return PK_OK;
}

template <int D, int ALGO, bool KPB>
int launch_one(const pk_problem& p, const Layout& L, cudaStream_t st, const DebugDump* dump) {
  if (dump && dump->ptr) return launch_one_impl<D, ALGO, KPB, 2, 1>(p, L, st, dump);
  if (dump && dump->timeline) return launch_one_impl<D, ALGO, KPB, 2, 2>(p, L, st, dump);
  if (dump && dump->skip_key_tile >= 0) return launch_one_impl<D, ALGO, KPB, 2, 3>(p, L, st, dump);
  return p.is_causal ? launch_one_impl<D, ALGO, KPB, 1, 0>(p, L, st, dump) : launch_one_impl<D, ALGO, KPB, 0, 0>(p, L, st, dump);
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
