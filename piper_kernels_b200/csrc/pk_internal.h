// Internal declarations shared by the translation units of libpiper_b200.so.
#pragma once

#include <cuda_runtime.h>

#include <utility>
#include <stddef.h>
#include <stdint.h>

#include "../../include/piper_b200.h"

namespace pk {

constexpr int kQTile = 128;       // query rows per CTA of the fused kernel
constexpr int kKeyTile = 64;      // keys per softmax tile (part of the numerics)
constexpr int kStatChunkRows = 512;  // rows per partial column reduction
constexpr float kLog2e = 1.4426950408889634f;

enum Algo : int { kPiper = 0, kSage = 1 };

// Byte offsets of every intermediate inside the caller's workspace.
struct Layout {
  int BH, D, Sq, Sk, sq_pad, sk_pad, chunks;
  int q_groups, k_groups;  // entries per head of the group-scale arrays
  // Heads with few query tiles (non-causal): the key tiles of every query tile are split over
  // `splits` CTAs of `tiles_per_split` tiles each, which leave un-normalised partial results in
  // `partial`; a merge kernel combines them.  splits == 1: no split.
  int splits, tiles_per_split;
  size_t status, k_mean, v_mean, k_part, v_part, q_codes, k_codes, v_codes, q_gscale, k_gscale,
      v_scale, q_mul, k_mul, k_add, k_inv, range, keys_alt, idx_a, idx_b, partial, total;
};

constexpr int kSplitBelowQueryTiles = 8;  // heads of up to 1024 query rows are candidates
constexpr int kCtasPerSmallHead = 16;     // CTAs such a head should contribute
constexpr int kMaxKeySplits = 8;
constexpr int kMinTilesPerSplit = 4;  // a CTA's pipeline needs a few tiles to fill
inline int partial_row_floats(int head_dim) { return head_dim + 4; }  // numerators, running max, denominator, padding

Layout make_layout(const pk_problem& p, Algo algo);

// Sets the thread-local error message and returns `code`.
int fail(int code, const char* fmt, ...);
const char* cuda_err(cudaError_t e);

// Argument checks shared by every entry point (does not touch the device).
int validate(const pk_problem* p, Algo algo, bool need_workspace);

// Prepass launchers (prepass.cu).  All asynchronous on `stream`.  `parts` selects what is
// quantised: the key/value side (statistics, key order, K and V codes, per-key vectors), the
// query side (Q codes and row multipliers), or both.
enum : int { kPrepassKV = 1, kPrepassQ = 2, kPrepassAll = 3 };
int launch_prepass(const pk_problem& p, const Layout& L, Algo algo, cudaStream_t stream, int parts);

// K and V sequence means with the partial sums in the library's own static device array
// (prepass.cu).  The caller has validated `p` and made p.device current.
int kv_means_static(const pk_problem& p, float* k_mean, float* v_mean);

// Fused kernels (fused_attention.cu).
struct DebugDump {
  void* ptr;        // first-tile intermediates (may be null)
  int bh, q_tile;   // which CTA
  void* timeline;   // per-role clock stamps (may be null)
  int timeline_tiles;
  int skip_key_tile;  // >= 0: stalled-wait drill, the producer leaves out this key tile's copy
};

// Device-visible address of this device's fault word: one pinned, mapped host int that a fused
// kernel writes its wait-site code to when it abandons a wait, so that the host can notice on its
// next call without synchronising.  Created on first use per device (p.device current); nullptr
// when the allocation is refused (the kernels then only write the workspace status words).
int32_t* fault_word_device_ptr(int device);
int launch_fused(const pk_problem& p, const Layout& L, Algo algo, cudaStream_t stream,
                 const DebugDump* dump);

template <typename T>
inline T* at(const pk_problem& p, size_t off) {
  return reinterpret_cast<T*>(static_cast<char*>(p.workspace) + off);
}

#ifdef __CUDACC__
// Launch with programmatic stream serialisation: the kernel may be set up and start while its
// predecessor in the stream is still draining, which hides most of the launch latency between the
// library's back-to-back kernels (a call is eight launches; small problems are bound by them).
// Every kernel launched this way calls cudaGridDependencySynchronize() before it touches memory:
// that returns once the predecessor has completed and its writes are visible.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<Args>(args))...);
}
#endif

}  // namespace pk
