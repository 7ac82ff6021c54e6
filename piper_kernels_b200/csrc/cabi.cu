// extern "C" surface of libpiper_b200.so (declared in include/piper_b200.h): argument checks,
// workspace layout, and the prepare / run orchestration that replaces the reference's Python
// host code (piper/triton.py:1054-1289, sage2pp/triton.py:446-679).

#include <math.h>
#include <stdarg.h>

#include <atomic>
#include <mutex>
#include <stdio.h>
#include <string.h>

#include "pk_internal.h"

namespace pk {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

const char* cuda_err(cudaError_t e) { return cudaGetErrorString(e); }

static size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

Layout make_layout(const pk_problem& p, Algo algo) {
  Layout L{};
  L.BH = p.batch * p.heads;
  L.D = p.head_dim;
  L.Sq = p.q_len;
  L.Sk = p.kv_len;
  L.sq_pad = (p.q_len + kQTile - 1) / kQTile * kQTile;
  L.sk_pad = (p.kv_len + kKeyTile - 1) / kKeyTile * kKeyTile;
  L.chunks = (p.kv_len + kStatChunkRows - 1) / kStatChunkRows;
  const bool per_thread = p.qk_granularity == PK_QK_PER_THREAD;
  L.q_groups = per_thread ? p.q_len : (p.q_len + 31) / 32;
  L.k_groups = per_thread ? p.kv_len : (p.kv_len + 63) / 64;
  const size_t BH = L.BH, D = L.D;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off = align256(off + bytes);
    return o;
  };
  L.status = take(64);
  L.k_mean = take(BH * D * 4);
  L.v_mean = take(BH * D * 4);
  L.k_part = take(BH * L.chunks * D * 8);
  L.v_part = take(BH * L.chunks * D * 8);
  L.q_codes = take(BH * L.sq_pad * D);
  L.k_codes = take(BH * L.sk_pad * D);
  L.v_codes = take(BH * D * L.sk_pad);
  L.q_gscale = take(BH * L.q_groups * 4);
  L.k_gscale = take(BH * L.k_groups * 4);
  const size_t vs_elems = (algo == kSage) ? BH * D : BH * static_cast<size_t>(L.Sk);
  L.v_scale = take(vs_elems * 4);
  L.q_mul = take(BH * L.sq_pad * 4);
  L.k_mul = take(BH * L.sk_pad * 4);
  L.k_add = take(BH * L.sk_pad * 4);
  L.k_inv = take(BH * L.sk_pad * 4);
  // Key-split policy: the counterpart of the reference's select_query_block (attention/scheduling.py:7-19),
  // which shrinks the query tile until every SM has a CTA.  Here the query tile stays 128 rows and, for
  // heads with few query tiles, the keys are split so that a head contributes about 16 CTAs.  The count
  // depends on the head's own shape only, never on batch*heads: a head's result is bit-identical
  // whichever other heads share its call (and however heads are sharded over GPUs).  Piper only: its
  // probability codes depend on a tile's own maximum, so a split changes nothing but the order of the
  // FP32 sums; Sage quantises probabilities against the running maximum, which a split would restart.
  L.splits = 1;
  L.tiles_per_split = L.sk_pad / kKeyTile;
  {
    const int n_qt = L.sq_pad / kQTile, n_all = L.sk_pad / kKeyTile;
    if (algo == kPiper && !p.is_causal && n_qt <= kSplitBelowQueryTiles) {
      int want = kCtasPerSmallHead / n_qt;
      if (want > kMaxKeySplits) want = kMaxKeySplits;
      if (want > n_all / kMinTilesPerSplit) want = n_all / kMinTilesPerSplit;
      if (want >= 2) {
        L.tiles_per_split = (n_all + want - 1) / want;
        L.splits = (n_all + L.tiles_per_split - 1) / L.tiles_per_split;  // no empty split
      }
    }
  }
  L.partial = 0;
  if (L.splits > 1) L.partial = take(BH * L.sq_pad * static_cast<size_t>(L.splits) * partial_row_floats(L.D) * 4);
  if (algo == kPiper && p.sort_value_rows) {
    L.range = take(BH * L.Sk * 4);
    L.keys_alt = take(BH * L.Sk * 4);
    L.idx_a = take(BH * L.Sk * 4);
    L.idx_b = take(BH * L.Sk * 4);
  }
  L.total = off;
  return L;
}

constexpr int kMaxDevices = 64;

static int device_major(int device) {
  // 0 = not yet queried; concurrent first calls store the same value
  static std::atomic<int> cache[kMaxDevices];
  if (device < 0 || device >= kMaxDevices) return -1;
  int major = cache[device].load(std::memory_order_acquire);
  if (major == 0) {
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess || major <= 0) return -1;
    cache[device].store(major, std::memory_order_release);
  }
  return major;
}

namespace {
struct FaultWord {
  std::once_flag once;
  int32_t* host = nullptr;
  int32_t* dev = nullptr;
};
FaultWord g_fault[kMaxDevices];

FaultWord* fault_word(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  FaultWord& f = g_fault[device];
  std::call_once(f.once, [&f] {
    void* h = nullptr;
    if (cudaHostAlloc(&h, sizeof(int32_t), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
      cudaGetLastError();
      return;
    }
    *static_cast<volatile int32_t*>(h) = 0;
    void* d = nullptr;
    if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
      cudaGetLastError();
      cudaFreeHost(h);
      return;
    }
    f.host = static_cast<int32_t*>(h);
    f.dev = static_cast<int32_t*>(d);
  });
  return &f;
}
}  // namespace

int32_t* fault_word_device_ptr(int device) {
  FaultWord* f = fault_word(device);
  return f ? f->dev : nullptr;
}

int validate(const pk_problem* p, Algo algo, bool need_workspace) {
  const char* name = algo == kPiper ? "piper_attention" : "sage_attention_2pp";
  if (!p) return fail(PK_ERR_BAD_ARG, "%s: null problem", name);
  if (p->batch <= 0 || p->heads <= 0) return fail(PK_ERR_BAD_ARG, "%s: batch and heads must be positive", name);
  if (p->q_len <= 0 || p->kv_len <= 0) return fail(PK_ERR_BAD_ARG, "%s does not accept empty query or key sequences", name);
  if (p->head_dim != 64 && p->head_dim != 128)
    return fail(PK_ERR_BAD_ARG, "%s supports head dimensions 64 and 128, got %d", name, p->head_dim);
  if (p->in_dtype != PK_F16 && p->in_dtype != PK_BF16) return fail(PK_ERR_BAD_ARG, "%s inputs must be float16 or bfloat16", name);
  if (p->out_dtype != p->in_dtype && p->out_dtype != PK_F32)
    return fail(PK_ERR_BAD_ARG, "%s output dtype must equal the input dtype or be PK_F32", name);
  if (p->is_causal && p->q_len != p->kv_len)
    return fail(PK_ERR_BAD_ARG, "causal %s requires equal query and key lengths, got %d/%d", name, p->q_len, p->kv_len);
  if (!(p->scale > 0.f) || !isfinite(p->scale)) return fail(PK_ERR_BAD_ARG, "%s scale must be finite and positive", name);
  if (p->qk_granularity != PK_QK_PER_BLOCK && p->qk_granularity != PK_QK_PER_THREAD)
    return fail(PK_ERR_BAD_ARG, "%s: unknown Q/K quantization granularity %d", name, p->qk_granularity);
  if (algo == kPiper && p->sort_value_rows) {
    if (p->is_causal) return fail(PK_ERR_BAD_ARG, "value-row ordering is valid only for non-causal attention");
    if (!p->center_value || p->qk_granularity != PK_QK_PER_BLOCK)
      return fail(PK_ERR_BAD_ARG, "value-row ordering requires centered non-causal grouped-QK attention");
  }
  if (!p->q || !p->k || !p->v) return fail(PK_ERR_BAD_ARG, "%s: null input pointer", name);
  if (static_cast<int64_t>(p->batch) * p->heads > 65535)
    return fail(PK_ERR_BAD_ARG, "%s: batch*heads must not exceed 65535 (got %lld); split the call", name,
                static_cast<long long>(p->batch) * p->heads);
  if (static_cast<int64_t>(p->batch) * p->heads * (static_cast<int64_t>(p->q_len) + 127) >= (1ll << 31) ||
      static_cast<int64_t>(p->batch) * p->heads * (static_cast<int64_t>(p->kv_len) + 63) >= (1ll << 31))
    return fail(PK_ERR_BAD_ARG, "%s: batch*heads*sequence must stay below 2^31 rows", name);
  if (need_workspace) {
    if (!p->out) return fail(PK_ERR_BAD_ARG, "%s: null output pointer", name);
    if (!p->workspace || (reinterpret_cast<uintptr_t>(p->workspace) & 255))
      return fail(PK_ERR_WORKSPACE, "%s: workspace must be a 256-byte aligned device pointer", name);
    const Layout L = make_layout(*p, algo);
    if (p->workspace_bytes < L.total)
      return fail(PK_ERR_WORKSPACE, "%s: workspace too small: %llu bytes given, %llu needed", name,
                  static_cast<unsigned long long>(p->workspace_bytes), static_cast<unsigned long long>(L.total));
    if (reinterpret_cast<uintptr_t>(p->out) & 15) return fail(PK_ERR_BAD_ARG, "%s: output must be 16-byte aligned", name);
  }
  return PK_OK;
}

namespace {

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int dev) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != dev) {
      err = cudaSetDevice(dev);
      switched = err == cudaSuccess;
    }
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

int check_arch(const pk_problem* p) {
  const int major = device_major(p->device);
  if (major < 0) return fail(PK_ERR_CUDA, "cannot query device %d", p->device);
  if (major != 10) return fail(PK_ERR_UNSUPPORTED_ARCH, "device %d has compute capability %d.x; this library is built for sm_100a only", p->device, major);
  return PK_OK;
}

void fill_views(const pk_problem& p, const Layout& L, Algo algo, pk_views* v) {
  memset(v, 0, sizeof(*v));
  v->q_codes = at<int8_t>(p, L.q_codes);
  v->k_codes = at<int8_t>(p, L.k_codes);
  v->v_codes_t = at<uint8_t>(p, L.v_codes);
  v->q_group_scale = at<float>(p, L.q_gscale);
  v->k_group_scale = at<float>(p, L.k_gscale);
  v->v_scale = at<float>(p, L.v_scale);
  v->k_mean = at<float>(p, L.k_mean);
  v->v_mean = at<float>(p, L.v_mean);
  v->order = (algo == kPiper && p.sort_value_rows) ? at<int32_t>(p, L.idx_a) : nullptr;
  v->q_row_mul = at<float>(p, L.q_mul);
  v->k_col_mul = at<float>(p, L.k_mul);
  v->k_col_add = at<float>(p, L.k_add);
  v->k_col_inv = at<float>(p, L.k_inv);
  v->status = at<int32_t>(p, L.status);
  v->sq_pad = L.sq_pad;
  v->sk_pad = L.sk_pad;
}

int workspace_bytes(const pk_problem* p, Algo algo, uint64_t* bytes) {
  g_err[0] = 0;
  if (!bytes) return fail(PK_ERR_BAD_ARG, "null size pointer");
  const int rc = validate(p, algo, false);
  if (rc) return rc;
  *bytes = make_layout(*p, algo).total;
  return PK_OK;
}

int prepare(const pk_problem* p, Algo algo, pk_views* views, int parts = kPrepassAll) {
  g_err[0] = 0;
  int rc = validate(p, algo, true);
  if (rc) return rc;
  DeviceGuard g(p->device);
  if (g.err != cudaSuccess) return fail(PK_ERR_CUDA, "cudaSetDevice(%d): %s", p->device, cuda_err(g.err));
  if ((rc = check_arch(p))) return rc;
  const Layout L = make_layout(*p, algo);
  if ((rc = launch_prepass(*p, L, algo, static_cast<cudaStream_t>(p->stream), parts))) return rc;
  if (views) fill_views(*p, L, algo, views);
  return PK_OK;
}

int run(const pk_problem* p, Algo algo, const DebugDump* dump) {
  g_err[0] = 0;
  int rc = validate(p, algo, true);
  if (rc) return rc;
  DeviceGuard g(p->device);
  if (g.err != cudaSuccess) return fail(PK_ERR_CUDA, "cudaSetDevice(%d): %s", p->device, cuda_err(g.err));
  if ((rc = check_arch(p))) return rc;
  const Layout L = make_layout(*p, algo);
  return launch_fused(*p, L, algo, static_cast<cudaStream_t>(p->stream), dump);
}

}  // namespace
}  // namespace pk

using namespace pk;

extern "C" {

PK_API int pk_version(void) { return PK_ABI_VERSION; }
PK_API const char* pk_last_error(void) { return g_err; }

PK_API int pk_piper_workspace_bytes(const pk_problem* p, uint64_t* bytes) { return workspace_bytes(p, kPiper, bytes); }
PK_API int pk_piper_prepare(const pk_problem* p, pk_views* views) { return prepare(p, kPiper, views); }
PK_API int pk_piper_prepare_kv(const pk_problem* p, pk_views* views) { return prepare(p, kPiper, views, kPrepassKV); }
PK_API int pk_piper_prepare_q(const pk_problem* p, pk_views* views) { return prepare(p, kPiper, views, kPrepassQ); }
PK_API int pk_piper_run(const pk_problem* p) { return run(p, kPiper, nullptr); }
PK_API int pk_piper_attention_fwd(const pk_problem* p) {
  const int rc = prepare(p, kPiper, nullptr);
  return rc ? rc : run(p, kPiper, nullptr);
}

PK_API int pk_sage2pp_workspace_bytes(const pk_problem* p, uint64_t* bytes) { return workspace_bytes(p, kSage, bytes); }
PK_API int pk_sage2pp_prepare(const pk_problem* p, pk_views* views) { return prepare(p, kSage, views); }
PK_API int pk_sage2pp_prepare_kv(const pk_problem* p, pk_views* views) { return prepare(p, kSage, views, kPrepassKV); }
PK_API int pk_sage2pp_prepare_q(const pk_problem* p, pk_views* views) { return prepare(p, kSage, views, kPrepassQ); }
PK_API int pk_sage2pp_run(const pk_problem* p) { return run(p, kSage, nullptr); }
PK_API int pk_sage2pp_attention_fwd(const pk_problem* p) {
  const int rc = prepare(p, kSage, nullptr);
  return rc ? rc : run(p, kSage, nullptr);
}

PK_API int pk_device_status(const pk_problem* p, int32_t status[16]) {
  g_err[0] = 0;
  if (!p || !status || !p->workspace) return fail(PK_ERR_BAD_ARG, "pk_device_status: null argument");
  DeviceGuard g(p->device);
  if (g.err != cudaSuccess) return fail(PK_ERR_CUDA, "cudaSetDevice(%d): %s", p->device, cuda_err(g.err));
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(p->stream));
  if (e != cudaSuccess) return fail(PK_ERR_CUDA, "stream synchronize: %s", cuda_err(e));
  e = cudaMemcpy(status, p->workspace, 16 * sizeof(int32_t), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail(PK_ERR_CUDA, "status copy: %s", cuda_err(e));
  if (status[0] != 0) return fail(PK_ERR_DEVICE_STATUS, "a fused kernel abandoned wait site %d", status[0]);
  return PK_OK;
}

PK_API int pk_kv_means_static(const pk_problem* p, float* k_mean, float* v_mean) {
  g_err[0] = 0;
  int rc = validate(p, kPiper, false);
  if (rc) return rc;
  if (!k_mean || !v_mean) return fail(PK_ERR_BAD_ARG, "pk_kv_means_static: null output pointer");
  DeviceGuard g(p->device);
  if (g.err != cudaSuccess) return fail(PK_ERR_CUDA, "cudaSetDevice(%d): %s", p->device, cuda_err(g.err));
  if ((rc = check_arch(p))) return rc;
  return kv_means_static(*p, k_mean, v_mean);
}

PK_API int pk_debug_first_tile(const pk_problem* p, int sage, int bh, int q_tile, void* dump) {
  if (!dump) return fail(PK_ERR_BAD_ARG, "pk_debug_first_tile: null dump pointer");
  const DebugDump d{dump, bh, q_tile, nullptr, 0, -1};
  return run(p, sage ? kSage : kPiper, &d);
}

PK_API int pk_debug_timeline(const pk_problem* p, int sage, int bh, int q_tile, void* stamps, int max_tiles) {
  if (!stamps || max_tiles <= 0) return fail(PK_ERR_BAD_ARG, "pk_debug_timeline: null buffer");
  const DebugDump d{nullptr, bh, q_tile, stamps, max_tiles, -1};
  return run(p, sage ? kSage : kPiper, &d);
}

PK_API int pk_debug_stalled_wait(const pk_problem* p, int sage, int skip_key_tile) {
  if (skip_key_tile < 0) return fail(PK_ERR_BAD_ARG, "pk_debug_stalled_wait: key tile index must be >= 0");
  const DebugDump d{nullptr, -1, -1, nullptr, 0, skip_key_tile};
  return run(p, sage ? kSage : kPiper, &d);
}

PK_API int pk_poll_device_fault(int device, int32_t* code) {
  g_err[0] = 0;
  if (!code) return fail(PK_ERR_BAD_ARG, "pk_poll_device_fault: null argument");
  *code = 0;
  if (device < 0 || device >= kMaxDevices) return fail(PK_ERR_BAD_ARG, "pk_poll_device_fault: bad device %d", device);
  // The word exists only after a launch on this device; nothing to report before that.
  FaultWord& f = g_fault[device];
  if (f.host == nullptr) return PK_OK;
  const int32_t v = __atomic_exchange_n(f.host, 0, __ATOMIC_ACQ_REL);
  *code = v;
  if (v != 0) return fail(PK_ERR_DEVICE_STATUS, "an earlier fused kernel on device %d abandoned wait site %d; its output rows were filled with NaN", device, v);
  return PK_OK;
}

}  // extern "C"
