/* piper_b200.h — C ABI of libpiper_b200.so: fused quantized attention forward for NVIDIA B200
 * (sm_100a).  Plain pointers and sizes only; no torch types.  All entry points are
 * re-entrant, launch on the caller's stream of the caller's device, never allocate device
 * memory and never synchronise (except pk_device_status, which the caller asks for).  The one
 * allocation the library ever makes is four bytes of pinned host memory per device, at the
 * first fused-kernel launch on that device (the fault word read by pk_poll_device_fault).
 *
 * The library replaces, for this one path, the operators that the reference project
 * (Boffee/piper-kernels) registers as
 *   piper_kernels::piper_attention(query, key, value, scale, is_causal, center_value)
 *       src/piper_kernels/attention/piper/triton.py:1319-1348
 *   piper_kernels::sage_attention_2pp(query, key, value, scale, is_causal)
 *       src/piper_kernels/attention/sage2pp/triton.py:434-443, 682-690
 * and the host orchestration behind them (prepare, then launch):
 *   _prepare_piper_attention / _launch_piper_attention   piper/triton.py:1054-1289
 *   _run_sage_attention_2pp                               sage2pp/triton.py:446-679
 */
#ifndef PIPER_B200_H
#define PIPER_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PK_ABI_VERSION 1

#if defined(__GNUC__)
#define PK_API __attribute__((visibility("default")))
#else
#define PK_API
#endif

/* return codes */
#define PK_OK 0
#define PK_ERR_BAD_ARG 1          /* shape / dtype / pointer / alignment rejected before launch */
#define PK_ERR_UNSUPPORTED_ARCH 2 /* device is not compute capability 10.x */
#define PK_ERR_WORKSPACE 3        /* workspace missing or smaller than pk_*_workspace_bytes */
#define PK_ERR_CUDA 4             /* a CUDA runtime / driver call failed (message has details) */
#define PK_ERR_DEVICE_STATUS 5    /* a kernel gave up a bounded wait; see pk_device_status */

/* element types */
#define PK_F16 0
#define PK_BF16 1
#define PK_F32 2 /* output only: un-rounded result for parity checks */

/* Q/K scale granularity (reference: qk_quantization="per_warp" | "per_thread",
 * attention/kernels/qk_quantization/int8/sage/reference.py:20-74) */
#define PK_QK_PER_BLOCK 0  /* one scale per 32 query rows / 64 key rows */
#define PK_QK_PER_THREAD 1 /* SageAttention's interleaved row groups */

/* One attention call.  Tensors are [batch, heads, sequence, head_dim] with a contiguous head
 * dimension; strides are in elements for batch, head and sequence.  q/k/v are borrowed and
 * never written.  `out` is contiguous [batch, heads, q_len, head_dim].
 * Limits: batch*heads <= 65535 (it is a grid dimension; split larger calls over the batch) and
 * batch*heads*(sequence rounded up to a tile) < 2^31 rows. */
typedef struct pk_problem {
  int32_t batch, heads, q_len, kv_len, head_dim; /* head_dim 64 or 128 */
  int32_t in_dtype;                              /* PK_F16 | PK_BF16 */
  int32_t out_dtype;                             /* in_dtype, or PK_F32 */
  int32_t is_causal;                             /* requires q_len == kv_len */
  int32_t center_value;                          /* piper: subtract the sequence mean of V */
  int32_t sort_value_rows;                       /* piper: centred-row-range key order */
  int32_t qk_granularity;                        /* PK_QK_PER_BLOCK | PK_QK_PER_THREAD */
  float scale;                                   /* softmax scale, finite and > 0 */
  const void* q;
  const void* k;
  const void* v;
  int64_t q_stride[3], k_stride[3], v_stride[3]; /* batch, head, sequence (elements) */
  void* out;
  const float* k_mean_override; /* optional [batch*heads, head_dim] f32 device pointers:  */
  const float* v_mean_override; /* use these means instead of computing them              */
  void* workspace;              /* device scratch, 256-byte aligned                       */
  uint64_t workspace_bytes;
  int32_t device; /* CUDA device ordinal that owns every pointer */
  void* stream;   /* cudaStream_t */
} pk_problem;

/* Device pointers into the workspace after a prepare call (for parity tests and for callers
 * that re-use quantised K/V).  Shapes: BH = batch*heads, Sq_pad = q_len rounded up to 128,
 * Sk_pad = kv_len rounded up to 64.  Padding rows hold zero codes. */
typedef struct pk_views {
  int8_t* q_codes;        /* [BH, Sq_pad, D]                                             */
  int8_t* k_codes;        /* [BH, Sk_pad, D]  (rows in sorted order when sorting)        */
  uint8_t* v_codes_t;     /* [BH, D, Sk_pad]  piper: int8; sage: E4M3                    */
  float* q_group_scale;   /* per-block: [BH, ceil(q_len/32)]; per-thread: [BH, q_len]    */
  float* k_group_scale;   /* per-block: [BH, ceil(kv_len/64)]; per-thread: [BH, kv_len]  */
  float* v_scale;         /* piper: [BH, kv_len] per key; sage: [BH, D] per channel      */
  float* k_mean;          /* [BH, D]                                                     */
  float* v_mean;          /* [BH, D] (zeros when not centring; unused by sage)           */
  int32_t* order;         /* [BH, kv_len] when sorting, else NULL                        */
  float* q_row_mul;       /* [BH, Sq_pad] q scale * softmax scale * log2(e)              */
  float* k_col_mul;       /* [BH, Sk_pad] per-key K scale                                */
  float* k_col_add;       /* [BH, Sk_pad] piper: log2(v scale); sage: 0; padding: -inf   */
  float* k_col_inv;       /* [BH, Sk_pad] piper: 1 / v scale; padding 0                  */
  int32_t* status;        /* [16] device status words, zero when healthy                 */
  int32_t sq_pad, sk_pad;
} pk_views;

PK_API int pk_version(void);
/* Message of the last failing call on this thread ("" if none). */
PK_API const char* pk_last_error(void);

/* Piper attention.  Replaces _prepare_piper_attention + _launch_piper_attention
 * (piper/triton.py:1054-1289) behind piper_kernels::piper_attention (:1319-1336). */
PK_API int pk_piper_workspace_bytes(const pk_problem* p, uint64_t* bytes);
PK_API int pk_piper_prepare(const pk_problem* p, pk_views* views); /* prepass only (piper/triton.py:1054-1236) */
/* Heads with at most 1024 query rows (non-causal): pk_piper_run splits every query tile's keys over up
 * to eight CTAs and merges their un-normalised rows in a second launch, so that short-query problems
 * fill the GPU (the role of the reference's select_query_block, attention/scheduling.py:7-19, which
 * shrinks the query tile instead).  The split depends on q_len and kv_len only, never on batch*heads:
 * a head's output is bit-identical whichever heads share its call.  The workspace size includes the
 * partial rows. */
PK_API int pk_piper_run(const pk_problem* p);                      /* fused kernel on a prepared workspace (:1239-1289) */
/* Prepared key/value reuse: the reference's benchmarks split every provider into prepare() and
 * run(prepared) (benchmarks/lib/attention_providers.py:201-216); cross-attention and diffusion
 * steps keep K/V and change only the queries.  pk_*_prepare_kv quantises the key/value side into
 * the workspace once (means, key order, K and V codes, per-key vectors: piper/triton.py:744-836,
 * 1119-1195; q is not read).  pk_*_prepare_q quantises a query batch of the same shape into the
 * same workspace (Q codes and row multipliers: piper/triton.py:839-973; k and v are not read but
 * must stay non-null).  Any sequence prepare_kv, then (prepare_q, run)* equals the same number
 * of full calls bit for bit. */
PK_API int pk_piper_prepare_kv(const pk_problem* p, pk_views* views);
PK_API int pk_piper_prepare_q(const pk_problem* p, pk_views* views);
PK_API int pk_piper_attention_fwd(const pk_problem* p);            /* prepare + run */

/* SageAttention2++ (8+8).  Replaces _run_sage_attention_2pp (sage2pp/triton.py:446-679)
 * behind piper_kernels::sage_attention_2pp (:434-443). */
PK_API int pk_sage2pp_workspace_bytes(const pk_problem* p, uint64_t* bytes);
PK_API int pk_sage2pp_prepare(const pk_problem* p, pk_views* views);
PK_API int pk_sage2pp_run(const pk_problem* p);
PK_API int pk_sage2pp_prepare_kv(const pk_problem* p, pk_views* views); /* K mean, V channel scale, K / V codes (sage2pp/triton.py:478-518, 631-647) */
PK_API int pk_sage2pp_prepare_q(const pk_problem* p, pk_views* views);  /* Q codes (sage2pp/triton.py:539-630) */
PK_API int pk_sage2pp_attention_fwd(const pk_problem* p);

/* Copies the 16 status words of the workspace to the host after synchronising the stream.
 * status[0] != 0 means a kernel abandoned a wait (the value says which one); the output rows of
 * the query tiles that gave up hold NaN. */
PK_API int pk_device_status(const pk_problem* p, int32_t status[16]);

/* Non-blocking check for the same condition, for callers that do not keep the workspace (the
 * torch operators): every fused kernel also writes its wait-site code into one pinned host word
 * per device; this call reads and clears it without touching the device or any stream.  Returns
 * PK_ERR_DEVICE_STATUS with *code != 0 when a kernel launched earlier on `device` gave up a
 * wait, PK_OK with *code == 0 otherwise.  The reference has no counterpart (its kernels cannot
 * give up a wait); it stands where the reference relies on CUDA's own launch errors. */
PK_API int pk_poll_device_fault(int32_t device, int32_t* code);

/* Debug aid for parity tests: runs the fused kernel and also copies the raw INT32 score tile
 * (first 64 keys, [128,64]), the packed probability codes ([128,64] bytes) and the raw PV
 * partial ([128, head_dim], int32 for piper / f32 for sage) of query tile `q_tile` of flattened
 * head `bh` into `dump` (device memory, 128*64*4 + 128*64 + 128*head_dim*4 bytes). */
PK_API int pk_debug_first_tile(const pk_problem* p, int sage, int bh, int q_tile, void* dump);

/* Profiling aid: runs the ordinary fused kernel and records, for the CTA of query tile `q_tile`
 * of flattened head `bh`, clock64() stamps of every warp role per key tile into `stamps`
 * (device memory, int64 [7 roles][max_tiles][8]; roles: the two softmax warpgroups, then
 * dequant, S-product issue, PV-product issue). */
PK_API int pk_debug_timeline(const pk_problem* p, int sage, int bh, int q_tile, void* stamps, int max_tiles);

/* Stalled-wait drill (test aid).  Runs the fused kernel on a prepared workspace with the copy of
 * key tile `skip_key_tile` left out by every CTA's producer and with every wait limited to about
 * 0.1 ms: the wait for that tile expires, every warp role unwinds, copies in flight are drained,
 * tensor memory is released and the kernel returns normally.  Afterwards pk_device_status and
 * pk_poll_device_fault report the wait site (22: the S-product issue warp waiting for a K tile),
 * the affected output rows hold NaN, and the device and context remain usable.  Nothing traps,
 * faults or spins without a limit. */
PK_API int pk_debug_stalled_wait(const pk_problem* p, int sage, int skip_key_tile);

/* K and V sequence means ([batch*heads, head_dim] f32 each, device memory) computed without a
 * workspace and without any allocation.  No counterpart in the reference: it exists for hosts
 * that cannot allocate device memory where they call the library (a frozen memory pool, a
 * runtime that hands a plug-in fixed buffers, an allocator whose state is being recorded).
 * The FP64 partial sums live in an 8 MiB array inside the library image, held by every device
 * that loads the library until the process exits.
 *   - Limit: batch*heads*ceil(kv_len/512)*head_dim <= 524288; larger problems are rejected with
 *     PK_ERR_BAD_ARG (use pk_piper_prepare with a workspace).
 *   - Only q-independent fields of `p` are used: batch, heads, kv_len, head_dim, in_dtype, k, v,
 *     their strides, device, stream (q_len/q/scale must still be valid).
 *   - The first call on a device looks up the array's device address; make that call before
 *     starting a stream capture.
 *   - All calls share the one array: calls that may overlap on the GPU (different streams) race.
 *     Nothing needs clearing between calls: each call overwrites every partial it reads.
 * Results are bit-identical to the k_mean / v_mean views of pk_piper_prepare with center_value=1. */
PK_API int pk_kv_means_static(const pk_problem* p, float* k_mean, float* v_mean);

#ifdef __cplusplus
}
#endif
#endif /* PIPER_B200_H */
