// Native executor for an inference pass over a chain of sparse convolutions.
//
// The reference runs a network layer by layer from Python (SparseSequential,
// spconv_triton/pytorch/modules.py:30-100): per layer one rulebook generation
// (ops.get_indice_pairs_implicit_gemm, a host read of the output count inside)
// and one GEMM (ops.implicit_gemm), dozens of small device allocations in
// between.  On B200 the kernels of a VoxelNet-sized forward take about half as
// long as that host work, so the pass is host-bound.  spc_sequence_forward runs
// the whole chain from one call: the same rulebook and GEMM entry points of
// this library, with every table, workspace and activation carved out of ONE
// caller-provided arena, on three streams:
//
//   chain   strided / transposed rulebooks, each of which needs the previous
//           one's output coordinates and one host read of its output count;
//   side    submanifold rulebooks (no host read), which only need the
//           coordinates of their level;
//   main    the GEMMs, each waiting (cudaStreamWaitEvent) for its rulebook.
//
// So the rulebook chain runs ahead of the GEMMs as far as its host reads allow
// and the submanifold rulebooks fill the gaps.  Results are the same tensors the
// layer-by-layer path produces (same kernels, same arguments).
#include <cstring>
#include <vector>

#include "common.cuh"
#include "rulebook_internal.cuh"

using namespace spc;

namespace {

constexpr int kMaxSeqLayers = 64;

struct EventPool {
  cudaEvent_t ev[kMaxSeqLayers + 2];
  bool ready = false;
};

// One pool per host thread and device: events are recorded and waited on inside one call only.
int events_for_current_device(cudaEvent_t** out) {
  static thread_local EventPool pools[kMaxDevices];
  const int dev = current_device_slot();
  if (dev < 0) return fail(SPC_ERR_CUDA, "sequence: no current device");
  EventPool& p = pools[dev];
  if (!p.ready) {
    for (auto& e : p.ev) SPC_CUDA_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    p.ready = true;
  }
  *out = p.ev;
  return SPC_OK;
}

struct Arena {
  char* base;
  size_t size, used = 0;
  bool overflow = false;
  // Offsets keep growing after an overflow so that the caller learns the size it needs.
  uint64_t take(size_t bytes) {
    const size_t at = used;
    used = align_up(used + std::max<size_t>(bytes, 16), 256);
    if (used > size) overflow = true;
    return at;
  }
  void* at(uint64_t off) const { return base + off; }
};

}  // namespace

extern "C" int spc_sequence_forward(const spc_seq_layer* layers, int n_layers, const int32_t* indices,
                                    const void* features, int64_t n_in, int dtype, void* arena_ptr,
                                    size_t arena_bytes, size_t* arena_needed, spc_seq_result* results,
                                    void* stream_main, void* stream_chain, void* stream_side) {
  if (!layers || n_layers <= 0 || n_layers > kMaxSeqLayers || !indices || !features || n_in <= 0 || !arena_ptr ||
      !arena_needed || !results || !stream_chain || !stream_side)
    return fail(SPC_ERR_INVALID_ARGUMENT, "sequence_forward: bad arguments");
  if (dtype != SPC_F16 && dtype != SPC_BF16)
    return fail(SPC_ERR_UNSUPPORTED, "sequence_forward: 16-bit features only");
  if ((reinterpret_cast<uintptr_t>(arena_ptr) & 255u) != 0)
    return fail(SPC_ERR_INVALID_ARGUMENT, "sequence_forward: the arena must be 256-byte aligned");
  cudaStream_t main = static_cast<cudaStream_t>(stream_main);
  cudaStream_t chain = static_cast<cudaStream_t>(stream_chain);
  cudaStream_t side = static_cast<cudaStream_t>(stream_side);
  cudaEvent_t* ev = nullptr;
  int rc = events_for_current_device(&ev);
  if (rc != SPC_OK) return rc;
  cudaEvent_t ev_input = ev[kMaxSeqLayers];

  Arena arena{static_cast<char*>(arena_ptr), arena_bytes};
  const size_t esize = dtype_size(dtype);
  const uint32_t split_word = 0xFFFFFFFFu;

  // the caller's stream has produced indices and features: the rulebook streams start after it
  SPC_CUDA_OK(cudaEventRecord(ev_input, main));
  SPC_CUDA_OK(cudaStreamWaitEvent(chain, ev_input, 0));
  SPC_CUDA_OK(cudaStreamWaitEvent(side, ev_input, 0));

  const int32_t* cur_indices = indices;   // coordinates of the current level
  int64_t cur_n = n_in;
  cudaEvent_t cur_indices_ready = ev_input;
  const void* cur_features = features;
  int cur_channels = layers[0].c_in;
  // the strided layer that produced the current level's coordinates: its output bitmap doubles as
  // the input bitmap of every rulebook generated from them
  RulebookProducer producer{nullptr, nullptr, 0};
  bool have_producer = false;

  for (int i = 0; i < n_layers; ++i) {
    const spc_seq_layer& L = layers[i];
    spc_seq_result& R = results[i];
    std::memset(&R, 0xFF, sizeof(R));  // every offset "absent" until set
    R.n_in = cur_n;
    if (L.c_in != cur_channels) return fail(SPC_ERR_INVALID_ARGUMENT, "sequence_forward: layer %d expects %d channels, gets %d", i, L.c_in, cur_channels);
    if (L.rulebook < 0 || L.rulebook > i) return fail(SPC_ERR_INVALID_ARGUMENT, "sequence_forward: layer %d names rulebook %d", i, L.rulebook);
    int kv = 1;
    for (int d = 0; d < L.geom.ndim; ++d) kv *= L.geom.ksize[d];
    if (kv < 1 || kv > 32) return fail(SPC_ERR_UNSUPPORTED, "sequence_forward: kernel volume %d (1..32 supported)", kv);
    const int kvp = (kv + 3) & ~3;

    if (L.rulebook == i) {
      // ---- generate this layer's rulebook --------------------------------------------------
      const bool subm = L.geom.subm != 0;
      cudaStream_t st = subm ? side : chain;
      if (subm) SPC_CUDA_OK(cudaStreamWaitEvent(side, cur_indices_ready, 0));
      const size_t ws_bytes = spc_rulebook_workspace_bytes(&L.geom, cur_n);
      if (ws_bytes == 0) return fail(SPC_ERR_INVALID_ARGUMENT, "sequence_forward: layer %d: geometry rejected", i);
      R.workspace = arena.take(ws_bytes);
      R.workspace_bytes = ws_bytes;
      if (arena.overflow) break;
      int64_t n_out = 0;
      rc = rulebook_prepare_chained(&L.geom, cur_indices, cur_n, arena.at(R.workspace), ws_bytes, &n_out,
                                    have_producer ? &producer : nullptr, st);
      if (rc != SPC_OK) return rc;
      R.n_out = n_out;
      if (n_out == 0) return fail(SPC_ERR_POINTS_VANISHED, "sequence_forward: layer %d has no output points", i);
      if (!subm) R.out_indices = arena.take(static_cast<size_t>(n_out) * (L.geom.ndim + 1) * 4);
      // the column-major table only if a layer that uses this rulebook reads it
      bool colmajor = false;
      for (int j = i; j < n_layers; ++j)
        if (layers[j].rulebook == i &&
            spc_conv_forward_needs_colmajor(layers[j].c_in, layers[j].c_out, kv, dtype, dtype, SPC_PREC_IEEE, SPC_GEMM_AUTO))
          colmajor = true;
      if (colmajor) R.pair_fwd = arena.take(static_cast<size_t>(kv) * n_out * 4);
      R.pair_fwd_rowmajor = arena.take(static_cast<size_t>(n_out) * kvp * 4);
      R.pair_mask = arena.take(static_cast<size_t>(n_out) * 4);
      R.mask_argsort = arena.take(static_cast<size_t>(n_out) * 4);
      R.num_per_loc = arena.take(static_cast<size_t>(kv) * 4);
      if (arena.overflow) break;
      SPC_CUDA_OK(cudaMemsetAsync(arena.at(R.num_per_loc), 0, static_cast<size_t>(kv) * 4, st));
      rc = rulebook_igemm_chained(&L.geom, cur_indices, cur_n, n_out, arena.at(R.workspace), ws_bytes,
                                  subm ? nullptr : static_cast<int32_t*>(arena.at(R.out_indices)),
                                  colmajor ? static_cast<int32_t*>(arena.at(R.pair_fwd)) : nullptr, nullptr,
                                  static_cast<int32_t*>(arena.at(R.pair_mask)),
                                  static_cast<int32_t*>(arena.at(R.mask_argsort)), nullptr, nullptr, &split_word, 1,
                                  /*do_sort=*/2, static_cast<int32_t*>(arena.at(R.pair_fwd_rowmajor)), nullptr,
                                  have_producer ? &producer : nullptr, st);
      if (rc != SPC_OK) return rc;
      R.masks_are_exact = rulebook_tile_key_applies(&L.geom, false, &split_word, 1) ? 0 : 1;
      SPC_CUDA_OK(cudaEventRecord(ev[i], st));
      if (!subm) {
        producer = RulebookProducer{&L.geom, arena.at(R.workspace), cur_n};
        have_producer = true;
        cur_indices = static_cast<const int32_t*>(arena.at(R.out_indices));
        cur_n = n_out;
        cur_indices_ready = ev[i];
      }
    } else {
      const spc_seq_result& G = results[L.rulebook];
      if (G.n_in != cur_n || layers[L.rulebook].geom.subm == 0)
        return fail(SPC_ERR_INVALID_ARGUMENT, "sequence_forward: layer %d cannot reuse the rulebook of layer %d", i, L.rulebook);
      R.n_out = G.n_out;
    }

    // ---- the GEMM, on the caller's stream, once its rulebook is there ---------------------------
    const spc_seq_result& G = results[L.rulebook];
    SPC_CUDA_OK(cudaStreamWaitEvent(main, ev[L.rulebook], 0));
    R.features = arena.take(static_cast<size_t>(R.n_out) * L.c_out * esize);
    if (arena.overflow) break;
    rc = spc_conv_forward(cur_features, L.weight, L.bias,
                          G.pair_fwd != UINT64_MAX ? static_cast<const int32_t*>(arena.at(G.pair_fwd)) : nullptr,
                          static_cast<const int32_t*>(arena.at(G.pair_fwd_rowmajor)),
                          kv > 1 ? static_cast<const int32_t*>(arena.at(G.mask_argsort)) : nullptr, arena.at(R.features),
                          R.n_in, R.n_out, L.c_in, L.c_out, kv, dtype, dtype, SPC_PREC_IEEE, SPC_GEMM_AUTO, L.scale,
                          L.shift, L.act, L.act_alpha, main);
    if (rc != SPC_OK) return rc;
    cur_features = arena.at(R.features);
    cur_channels = L.c_out;
  }

  *arena_needed = arena.used;
  // work queued on the rulebook streams must be over before the caller may free or reuse the arena
  // on its own stream: the caller's stream joins both
  SPC_CUDA_OK(cudaEventRecord(ev[kMaxSeqLayers + 1], chain));
  SPC_CUDA_OK(cudaStreamWaitEvent(main, ev[kMaxSeqLayers + 1], 0));
  SPC_CUDA_OK(cudaEventRecord(ev_input, side));
  SPC_CUDA_OK(cudaStreamWaitEvent(main, ev_input, 0));
  if (arena.overflow) {
    // a lower bound: the layers after the one that did not fit are not counted
    *arena_needed = arena.used * 2;
    return fail(SPC_ERR_WORKSPACE_TOO_SMALL, "sequence_forward: the arena holds %zu bytes, at least %zu are needed", arena_bytes, arena.used);
  }
  return SPC_OK;
}
