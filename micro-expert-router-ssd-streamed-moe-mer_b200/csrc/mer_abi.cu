// C-ABI layer: backend handle, HBM expert slot arena (VRAM tier), router table, dispatch.
// Host code only; kernels live in kernels_*.cu.  See include/mer_b200.h for the contract and
// the reference interfaces each entry point replaces.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <functional>
#include <mutex>
#include <new>
#include <unordered_map>
#include <vector>

#include "../../include/mer_b200.h"
#include "kernels.h"

#define MER_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t SLOT_HEADER_BYTES = 256;  // {epoch, expert id, payload bytes}; payload stays 256-B aligned
constexpr size_t SLOT_ALIGN = 4096;        // page-aligned slot stride (block_align of the reference's blobs)
constexpr size_t STAGE_BYTES = 16u << 20;  // two pinned staging buffers for pageable host blobs
constexpr uint32_t MAX_DIM = 1u << 20;

struct SlotHeader {  // written at the start of every occupied slot
  uint64_t epoch;
  uint32_t expert_id;
  uint32_t dtype;
  uint64_t payload_bytes;
};

struct Slot {
  bool used = false, anchor = false;
  uint32_t expert_id = MER_NONE;
  uint64_t generation = 0, last_use = 0;
};

struct RouterEntry {
  RouterDev dev{};
  float *d_w = nullptr, *d_cbias = nullptr, *d_lbias = nullptr;
  // steps either side of the MoE block (mer_layer_install)
  float *d_rms_w = nullptr, *d_shared_gate = nullptr;
  float rms_eps = 0.0f;
  uint32_t layer_flags = 0;
};

}  // namespace

struct mer_a2a_state;  // NCCL all-to-all mode (mer_abi_ep_nccl.inc)

struct mer_backend {
  mer_backend_cfg cfg{};
  mer_a2a_state *a2a = nullptr;
  int sm_count = 0;
  size_t expert_bytes = 0;
  cudaStream_t compute = nullptr, copy = nullptr;
  cudaEvent_t ev_compute_done = nullptr, ev_copy_done = nullptr, ev_stage[2] = {nullptr, nullptr};
  bool copy_pending = false;

  // VRAM tier
  uint8_t *arena = nullptr;
  size_t slot_stride = 0, n_slots = 0;
  std::vector<Slot> slots;
  std::unordered_map<uint32_t, size_t> id2slot;
  const uint8_t **d_expert_ptr = nullptr;  // device table: global id -> payload
  const uint8_t **h_expert_ptr = nullptr;  // pinned mirror
  uint8_t *h_stage[2] = {nullptr, nullptr};
  SlotHeader *h_hdr = nullptr;  // pinned, one per slot
  uint64_t tick = 0;

  // workspace
  uint32_t max_pairs = 0;
  float *d_x = nullptr, *d_out = nullptr, *d_h = nullptr, *d_y = nullptr, *d_pair_weight = nullptr, *d_logits = nullptr;
  uint32_t *d_pair_expert = nullptr, *d_group_expert = nullptr, *d_offsets = nullptr, *d_perm = nullptr;
  uint32_t *d_status = nullptr, *d_counters = nullptr, *d_group_count = nullptr;  // d_group_count: [2 x max_groups]
  float *d_xn = nullptr, *d_shared_scale = nullptr;  // RMSNorm'ed rows [max_tokens x D] and shared-expert gate scalars (allocated on first mer_layer_install)
  uint16_t *d_f16 = nullptr;
  void *d_stream_scratch = nullptr;
  void *d_gemm_scratch = nullptr;  // activation operand images of the tensor-core GEMM path
  size_t gemm_scratch_bytes = 0;
  uint32_t max_groups = 0, max_router_experts = 0;
  uint32_t *h_u32 = nullptr;  // pinned [max_pairs + 1]: ids up/down, status
  float *h_f32 = nullptr;     // pinned [max_pairs]
  float *d_dequant = nullptr;
  bool packed = false;          // slots hold the tile-major fragment layout (block-aligned shapes)
  uint8_t *d_raw_stage = nullptr;  // device copy of one flat blob, source of the repack at admission

  std::unordered_map<uint32_t, RouterEntry> routers;
  int kernel_path = 0;

  // pipelined host entry (mer_moe_layer_forward_submit / _wait): per slot its own device x / out and status copy
  struct AsyncSlot {
    float *d_x = nullptr, *d_out = nullptr;
    uint32_t *d_status = nullptr, *h_status = nullptr;
    cudaEvent_t ev_in = nullptr, ev_compute = nullptr, ev_out = nullptr;
    bool in_flight = false;
    uint32_t layer = 0;
    size_t pairs = 0;
  };
  AsyncSlot aslots[MER_ASYNC_SLOTS];
  cudaStream_t d2h = nullptr;

  // expert parallel (mer_ep_*): exchange buffer mapped by the peers, peers' buffers mapped here
  bool ep_on = false, ep_attached = false;
  EpDev ep{};
  mer_ep_cfg ep_cfg{};
  uint8_t *ep_buf = nullptr;
  size_t ep_bytes = 0, ep_off_w = 0;
  uint16_t *d_ep_owner = nullptr;       // placement table [max_experts] (mer_ep_set_placement), device copy
  std::vector<uint16_t> ep_owner_host;  // and host copy; empty = the contiguous rule
  void *ep_opened[MER_EP_MAX_WORLD] = {};  // mappings opened from IPC handles (closed at destroy)
  // captured launch sequences of mer_moe_layer_forward_device, replayed with one cudaGraphLaunch
  struct GraphEntry {
    uint32_t layer;
    size_t n_tokens;
    const void *x, *out, *ids, *w;
    cudaStream_t stream;
    cudaGraphExec_t exec;
    int launches;
  };
  std::vector<GraphEntry> graphs;
  bool graphs_ok = true;
  // Streams other than `compute` that device entry points were last enqueued on, each with an event recorded after
  // the call: an admission or a retire makes the copy stream wait for all of them before it touches a slot.
  struct UserStream {
    cudaStream_t stream;
    cudaEvent_t done;
    uint64_t last_use;
  };
  std::vector<UserStream> user_streams;
  // stage timing: sets of 5 events {start, after router, mid FFN, after FFN, after combine}
  bool timing_on = false;
  std::vector<cudaEvent_t> timing_events;
  size_t timing_used = 0;
  mer_stage_timings timing_acc{};
  std::mutex mu;
  mer_error_info err{};
  mer_counters ctr{};
};

namespace {

int fail(mer_backend *b, int kind, uint32_t layer, uint32_t expert, const char *fmt, ...) {
  if (b) {
    b->err.layer = layer;
    b->err.expert_id = expert;
    b->err.kind = kind;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(b->err.detail, sizeof b->err.detail, fmt, ap);
    va_end(ap);
  }
  return kind;
}

int cuda_fail(mer_backend *b, int kind, uint32_t layer, uint32_t expert, const char *what, cudaError_t e) {
  if (e == cudaErrorDevicesUnavailable || e == cudaErrorNoDevice || e == cudaErrorECCUncorrectable ||
      e == cudaErrorHardwareStackError || e == cudaErrorIllegalAddress || e == cudaErrorLaunchFailure)
    kind = MER_ERR_DEVICE_LOST;
  return fail(b, kind, layer, expert, "%s: %s", what, cudaGetErrorString(e));
}

#define CU(kind, what, call)                                          \
  do {                                                                \
    cudaError_t e__ = (call);                                         \
    if (e__ != cudaSuccess) return cuda_fail(b, kind, layer, expert, what, e__); \
  } while (0)

size_t block_bytes(int dtype) { return dtype == MER_DTYPE_Q4_0 ? MER_Q4_BLOCK_BYTES : MER_Q8_BLOCK_BYTES; }

MoeDispatch base_dispatch(mer_backend *b) {
  MoeDispatch d{};
  d.expert_ptr = b->d_expert_ptr;
  d.max_experts = b->cfg.max_experts;
  d.dtype = b->cfg.dtype;
  d.D = (uint32_t)b->cfg.d_model;
  d.F = (uint32_t)b->cfg.d_ff;
  d.pair_expert = b->d_pair_expert;
  d.pair_weight = b->d_pair_weight;
  d.group_expert = b->d_group_expert;
  d.offsets = b->d_offsets;
  d.perm = b->d_perm;
  d.group_count = b->d_group_count;
  d.group_cursor = b->d_group_count ? b->d_group_count + b->max_groups : nullptr;
  d.h = b->d_h;
  d.y = b->d_y;
  d.status = b->d_status;
  d.counters = b->d_counters;
  d.logits = b->d_logits;
  d.swiglu_limit = b->cfg.swiglu_limit;
  d.scratch_pairs = b->max_pairs;
  d.packed = b->packed ? 1 : 0;
  d.residual = nullptr;
  d.routed_slots = 0xFFFFFFFFu;
  return d;
}

// Uploads enqueued on the copy stream must land before the next kernel reads a slot.
cudaError_t order_after_copies(mer_backend *b, cudaStream_t s) {
  if (!b->copy_pending) return cudaSuccess;
  cudaError_t e = cudaStreamWaitEvent(s, b->ev_copy_done, 0);
  if (e == cudaSuccess && s == b->compute) b->copy_pending = false;
  return e;
}

constexpr size_t MAX_USER_STREAMS = 8;

// Records that work reading the slot arena was just enqueued on caller stream `s`.
cudaError_t note_stream_use(mer_backend *b, cudaStream_t s) {
  if (s == b->compute) return cudaSuccess;  // ordered through ev_compute_done
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return cudaSuccess;  // a call captured into the caller's own graph: the caller orders its replays against admissions
  }
  mer_backend::UserStream *slot = nullptr;
  for (auto &u : b->user_streams)
    if (u.stream == s) slot = &u;
  if (!slot) {
    if (b->user_streams.size() < MAX_USER_STREAMS) {
      cudaEvent_t ev;
      cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
      if (e != cudaSuccess) return e;
      b->user_streams.push_back({s, ev, 0});
      slot = &b->user_streams.back();
    } else {
      // more distinct streams than tracked: the least recently used one is synchronised and its entry reused
      slot = &b->user_streams[0];
      for (auto &u : b->user_streams)
        if (u.last_use < slot->last_use) slot = &u;
      cudaError_t e = cudaEventSynchronize(slot->done);
      if (e != cudaSuccess) return e;
      slot->stream = s;
    }
  }
  slot->last_use = ++b->tick;
  return cudaEventRecord(slot->done, s);
}

// Before the copy stream overwrites, repacks or unmaps a slot: everything already enqueued that may read the arena
// (the backend's compute stream and every tracked caller stream) must have finished.
cudaError_t copy_waits_for_readers(mer_backend *b) {
  cudaError_t e = cudaEventRecord(b->ev_compute_done, b->compute);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(b->copy, b->ev_compute_done, 0);
  for (auto &u : b->user_streams)
    if (e == cudaSuccess) e = cudaStreamWaitEvent(b->copy, u.done, 0);
  return e;
}

bool use_stream_path(mer_backend *b, const MoeDispatch &d) {
  if (b->kernel_path == 1) return false;
  return stream_ffn_supported(d.dtype, d.D, d.F) && b->d_stream_scratch != nullptr;
}

constexpr uint32_t GEMM_MIN_MEAN_TOKENS = 12;  // mean tokens per expert from which the tcgen05 GEMM path takes over (measured:
                                               // at a mean of 8-9 the streaming kernels are level or ahead, at 16 the GEMM kernels
                                               // win by 5 % on Mixtral-sized and by 50 % on Qwen3-sized experts)

// Chooses the kernel family of a dispatch and binds its scratch (call before the grouping kernel, which
// cuts the groups into passes of d.tokens_per_pass).
void bind_ffn(mer_backend *b, MoeDispatch &d) {
  d.gemm_bn = 0;
  if (!use_stream_path(b, d)) return;
  if (b->d_gemm_scratch && b->kernel_path != 2) {
    const uint32_t bn = gemm_pick_bn(d, b->kernel_path == 3 ? 1u : GEMM_MIN_MEAN_TOKENS);
    if (bn) {
      gemm_bind(d, b->d_stream_scratch, b->sm_count, bn);
      d.gemm_bn = bn;
      return;
    }
  }
  stream_bind(d, b->d_stream_scratch, b->sm_count);
}

cudaError_t run_ffn(mer_backend *b, MoeDispatch &d, cudaStream_t s, int *launches, cudaEvent_t ev_mid = nullptr) {
  d.y_parts = nullptr, d.y_nparts = 1;
  d.combined = 0;
  if (d.gemm_bn)
    return launch_ffn_gemm(d, b->d_gemm_scratch, b->gemm_scratch_bytes, std::max(b->cfg.max_tokens, b->max_pairs), b->sm_count, s, launches,
                           ev_mid);
  if (use_stream_path(b, d)) return launch_ffn_stream(d, b->d_stream_scratch, b->sm_count, s, launches, ev_mid);
  return launch_ffn_generic(d, s, launches, ev_mid);
}

constexpr size_t TIMING_SET = 5, TIMING_MAX_SETS = 4096;

// Returns the next set of 5 events, or null when timing is off or the ring is full.
cudaEvent_t *next_timing_set(mer_backend *b) {
  if (!b->timing_on || b->timing_used >= TIMING_MAX_SETS) return nullptr;
  size_t need = (b->timing_used + 1) * TIMING_SET;
  while (b->timing_events.size() < need) {
    cudaEvent_t e;
    if (cudaEventCreate(&e) != cudaSuccess) return nullptr;
    b->timing_events.push_back(e);
  }
  return &b->timing_events[b->timing_used++ * TIMING_SET];
}

void drain_timing(mer_backend *b) {
  for (size_t i = 0; i < b->timing_used; i++) {
    cudaEvent_t *e = &b->timing_events[i * TIMING_SET];
    if (cudaEventSynchronize(e[4]) != cudaSuccess) continue;
    float r = 0, gu = 0, dn = 0, cb = 0;
    cudaEventElapsedTime(&r, e[0], e[1]);
    bool have_mid = cudaEventQuery(e[2]) == cudaSuccess && cudaEventElapsedTime(&gu, e[1], e[2]) == cudaSuccess;
    if (have_mid) {
      cudaEventElapsedTime(&dn, e[2], e[3]);
    } else {
      cudaGetLastError();
      cudaEventElapsedTime(&gu, e[1], e[3]);
    }
    cudaEventElapsedTime(&cb, e[3], e[4]);
    b->timing_acc.samples++;
    b->timing_acc.router_gate_ms += r;
    b->timing_acc.expert_gate_up_kernel_ms += gu;
    b->timing_acc.expert_down_kernel_ms += dn;
    b->timing_acc.moe_weighted_combination_ms += cb;
    b->timing_acc.expert_compute_ms += gu + dn;
  }
  b->timing_used = 0;
}

void drop_graphs(mer_backend *b) {
  if (b->graphs.empty()) return;
  cudaDeviceSynchronize();
  for (auto &g : b->graphs) cudaGraphExecDestroy(g.exec);
  b->graphs.clear();
}

int check_device_status(mer_backend *b, uint32_t status, uint32_t layer, uint32_t expert) {
  b->err.device_status = status;
  if (status & MER_DEVSTAT_RESIDENCY_MISS)
    return fail(b, MER_ERR_RESIDENCY_MISS, layer, expert, "a routed expert has no current HBM slot (device status 0x%x)", status);
  if (status & MER_DEVSTAT_TIMEOUT)
    return fail(b, MER_ERR_TIMEOUT, layer, expert, "a bounded device-side wait expired (device status 0x%x)", status);
  if (status & MER_DEVSTAT_NONFINITE_ROUTER)
    return fail(b, MER_ERR_NUMERICAL, layer, expert, "non-finite router scores (device status 0x%x)", status);
  return MER_OK;
}

int validate_shape_args(mer_backend *b, uint32_t layer, uint32_t expert, size_t d_model, size_t d_ff) {
  if (d_model != b->cfg.d_model || d_ff != b->cfg.d_ff)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "shape %zux%zu does not match the backend's %llux%llu", d_model,
                d_ff, (unsigned long long)b->cfg.d_model, (unsigned long long)b->cfg.d_ff);
  return MER_OK;
}

// Host-side residency check for calls whose expert ids are known on the host
// (current_admission miss -> ResidencyMiss, backend/mod.rs:3870-3882).
int require_resident(mer_backend *b, uint32_t layer, uint32_t id) {
  auto it = b->id2slot.find(id);
  if (id >= b->cfg.max_experts || it == b->id2slot.end())
    return fail(b, MER_ERR_RESIDENCY_MISS, layer, id, "expert has no current logical GPU admission");
  b->slots[it->second].last_use = ++b->tick;
  return MER_OK;
}

void a2a_free(mer_backend *b);  // mer_abi_ep_nccl.inc

void free_all(mer_backend *b) {
  a2a_free(b);
  auto F = [](auto *&p) {
    if (p) cudaFree((void *)p);
    p = nullptr;
  };
  auto H = [](auto *&p) {
    if (p) cudaFreeHost((void *)p);
    p = nullptr;
  };
  for (auto &kv : b->routers) {
    F(kv.second.d_w);
    F(kv.second.d_cbias);
    F(kv.second.d_lbias);
    F(kv.second.d_rms_w);
    F(kv.second.d_shared_gate);
  }
  b->routers.clear();
  F(b->arena), F(b->d_expert_ptr), F(b->d_x), F(b->d_out), F(b->d_h), F(b->d_y), F(b->d_pair_weight), F(b->d_logits);
  F(b->d_pair_expert), F(b->d_group_expert), F(b->d_offsets), F(b->d_perm), F(b->d_status), F(b->d_counters), F(b->d_group_count);
  F(b->d_f16), F(b->d_stream_scratch), F(b->d_gemm_scratch), F(b->d_dequant), F(b->d_raw_stage), F(b->d_xn), F(b->d_shared_scale);
  H(b->h_expert_ptr), H(b->h_stage[0]), H(b->h_stage[1]), H(b->h_hdr), H(b->h_u32), H(b->h_f32);
  if (b->ev_compute_done) cudaEventDestroy(b->ev_compute_done);
  if (b->ev_copy_done) cudaEventDestroy(b->ev_copy_done);
  for (auto &e : b->ev_stage)
    if (e) cudaEventDestroy(e);
  for (auto &g : b->graphs) cudaGraphExecDestroy(g.exec);
  b->graphs.clear();
  for (auto &e : b->timing_events) cudaEventDestroy(e);
  b->timing_events.clear();
  for (auto &u : b->user_streams) cudaEventDestroy(u.done);
  b->user_streams.clear();
  for (auto &a : b->aslots) {
    F(a.d_x), F(a.d_out), F(a.d_status), H(a.h_status);
    if (a.ev_in) cudaEventDestroy(a.ev_in);
    if (a.ev_compute) cudaEventDestroy(a.ev_compute);
    if (a.ev_out) cudaEventDestroy(a.ev_out);
  }
  if (b->d2h) cudaStreamDestroy(b->d2h);
  for (auto &p : b->ep_opened)
    if (p) cudaIpcCloseMemHandle(p), p = nullptr;
  F(b->ep_buf);
  F(b->d_ep_owner);
  if (b->compute) cudaStreamDestroy(b->compute);
  if (b->copy) cudaStreamDestroy(b->copy);
}

// Picks a slot for (id, generation): reuse, free, or least-recently-used non-anchor victim
// (demand_admit_lru, expert_cache.rs:1281-1340: the anchor region is never touched).
int acquire_slot(mer_backend *b, uint32_t id, uint64_t generation, uint32_t flags, size_t *out, bool *already) {
  const uint32_t layer = 0, expert = id;
  *already = false;
  auto it = b->id2slot.find(id);
  if (it != b->id2slot.end()) {
    Slot &s = b->slots[it->second];
    if (generation < s.generation)
      return fail(b, MER_ERR_RESIDENCY_MISS, layer, expert, "physical GPU residency has a newer logical generation (%llu > %llu)",
                  (unsigned long long)s.generation, (unsigned long long)generation);
    if (generation == s.generation) {
      *already = true;
      *out = it->second;
      return MER_OK;
    }
    *out = it->second;  // newer generation replaces the payload in place
    return MER_OK;
  }
  size_t victim = SIZE_MAX;
  for (size_t i = 0; i < b->n_slots; i++)
    if (!b->slots[i].used) {
      victim = i;
      break;
    }
  if (victim == SIZE_MAX) {
    uint64_t best = UINT64_MAX;
    for (size_t i = 0; i < b->n_slots; i++)
      if (!b->slots[i].anchor && b->slots[i].last_use < best) best = b->slots[i].last_use, victim = i;
    if (victim == SIZE_MAX)
      return fail(b, MER_ERR_PHYSICAL_CAPACITY, layer, expert, "all %zu HBM slots hold anchor experts", b->n_slots);
    Slot &v = b->slots[victim];
    b->id2slot.erase(v.expert_id);
    b->h_expert_ptr[v.expert_id] = nullptr;
    cudaMemcpyAsync((void *)(b->d_expert_ptr + v.expert_id), (void *)(b->h_expert_ptr + v.expert_id), sizeof(void *),
                    cudaMemcpyHostToDevice, b->copy);
    v.used = false;
    b->ctr.evictions++;
  }
  (void)flags;
  *out = victim;
  return MER_OK;
}

// Fills `dst` with bytes [off, off + n) of the expert's gate||up||down stream; false = the source ran short.
using ChunkReader = std::function<bool(size_t off, size_t n, uint8_t *dst)>;

int admit_impl(mer_backend *b, uint32_t id, uint64_t generation, const void *blob, size_t bytes, uint32_t flags,
               bool from_device, const ChunkReader *reader = nullptr) {
  const uint32_t layer = 0, expert = id;
  if (!b || !blob) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null backend or blob");
  if (id >= b->cfg.max_experts)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "expert id %u outside the id space of %u", id, b->cfg.max_experts);
  // plan_expert_upload_q4_0 (backend/mod.rs:2482-2549): strict payload size; page padding after
  // the logical payload is allowed and never copied.
  if (bytes < b->expert_bytes)
    return fail(b, MER_ERR_UPLOAD, layer, expert, "blob has %zu bytes, need %zu for %llux%llu", bytes, b->expert_bytes,
                (unsigned long long)b->cfg.d_model, (unsigned long long)b->cfg.d_ff);
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_UPLOAD, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  // A slot (the victim's table entry included) may still be read by layers already enqueued: every write of this
  // admission, the eviction's table update first, is ordered after them.
  if (!(flags & MER_ADMIT_NO_READER_WAIT)) CU(MER_ERR_UPLOAD, "order the copy stream after the readers", copy_waits_for_readers(b));
  size_t si;
  bool already;
  int rc = acquire_slot(b, id, generation, flags, &si, &already);
  if (rc) return rc;
  Slot &s = b->slots[si];
  if (already) {
    s.last_use = ++b->tick;
    if (flags & MER_ADMIT_ANCHOR) s.anchor = true;
    return MER_OK;
  }
  uint8_t *slot_base = b->arena + si * b->slot_stride;
  uint8_t *payload = slot_base + SLOT_HEADER_BYTES;
  uint8_t *landing = b->packed ? b->d_raw_stage : payload;  // packed slots: land flat bytes in staging, then permute
  const uint8_t *src = static_cast<const uint8_t *>(blob);
  if (from_device) {
    if (b->packed)
      landing = const_cast<uint8_t *>(src);  // permute straight out of the caller's device buffer
    else
      CU(MER_ERR_UPLOAD, "cudaMemcpyAsync(D2D)", cudaMemcpyAsync(payload, src, b->expert_bytes, cudaMemcpyDeviceToDevice, b->copy));
  } else {
    cudaPointerAttributes attr{};
    bool pinned = !reader && cudaPointerGetAttributes(&attr, blob) == cudaSuccess && attr.type == cudaMemoryTypeHost;
    cudaGetLastError();
    if (pinned) {
      CU(MER_ERR_UPLOAD, "cudaMemcpyAsync(H2D pinned)",
         cudaMemcpyAsync(landing, src, b->expert_bytes, cudaMemcpyHostToDevice, b->copy));
    } else {
      int which = 0;
      for (size_t off = 0; off < b->expert_bytes; off += STAGE_BYTES, which ^= 1) {
        size_t n = std::min(STAGE_BYTES, b->expert_bytes - off);
        CU(MER_ERR_UPLOAD, "cudaEventSynchronize(stage)", cudaEventSynchronize(b->ev_stage[which]));
        if (reader) {  // e.g. pread from an expert file, straight into the pinned staging buffer
          if (!(*reader)(off, n, b->h_stage[which]))
            return fail(b, MER_ERR_UPLOAD, layer, expert, "the expert source ended before byte %zu of %zu", off + n, b->expert_bytes);
        } else {
          memcpy(b->h_stage[which], src + off, n);
        }
        CU(MER_ERR_UPLOAD, "cudaMemcpyAsync(H2D staged)",
           cudaMemcpyAsync(landing + off, b->h_stage[which], n, cudaMemcpyHostToDevice, b->copy));
        CU(MER_ERR_UPLOAD, "cudaEventRecord(stage)", cudaEventRecord(b->ev_stage[which], b->copy));
      }
    }
  }
  if (b->packed)
    CU(MER_ERR_UPLOAD, "repack kernel",
       launch_repack(b->cfg.dtype, landing, payload, (uint32_t)b->cfg.d_model, (uint32_t)b->cfg.d_ff, b->copy));
  SlotHeader *hdr = b->h_hdr + si;
  hdr->epoch = generation;
  hdr->expert_id = id;
  hdr->dtype = (uint32_t)b->cfg.dtype;
  hdr->payload_bytes = b->expert_bytes;
  CU(MER_ERR_UPLOAD, "cudaMemcpyAsync(header)", cudaMemcpyAsync(slot_base, hdr, sizeof(SlotHeader), cudaMemcpyHostToDevice, b->copy));
  b->h_expert_ptr[id] = payload;
  CU(MER_ERR_UPLOAD, "cudaMemcpyAsync(table)",
     cudaMemcpyAsync((void *)(b->d_expert_ptr + id), (void *)(b->h_expert_ptr + id), sizeof(void *), cudaMemcpyHostToDevice, b->copy));
  CU(MER_ERR_UPLOAD, "cudaEventRecord(copy)", cudaEventRecord(b->ev_copy_done, b->copy));
  b->copy_pending = true;
  s.used = true;
  s.anchor = (flags & MER_ADMIT_ANCHOR) != 0;
  s.expert_id = id;
  s.generation = generation;
  s.last_use = ++b->tick;
  b->id2slot[id] = si;
  b->ctr.expert_uploads++;
  b->ctr.expert_upload_bytes += b->expert_bytes;
  if (!(flags & MER_ADMIT_ASYNC)) CU(MER_ERR_UPLOAD, "cudaStreamSynchronize(copy)", cudaStreamSynchronize(b->copy));
  return MER_OK;
}

// Shared tail of the host entry points whose routing comes from the caller: upload ids and
// weights, group, run the FFN.  `single_group` = all pairs run the same expert.
int dispatch_given_routing(mer_backend *b, uint32_t layer, MoeDispatch &d, const uint32_t *ids, const float *weights,
                           size_t n_pairs, bool single_group, int *launches, bool combine_follows = false) {
  const uint32_t expert = n_pairs ? ids[0] : MER_NONE;
  memcpy(b->h_u32, ids, n_pairs * sizeof(uint32_t));
  for (size_t i = 0; i < n_pairs; i++) b->h_f32[i] = weights ? weights[i] : 1.0f;
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(ids)",
     cudaMemcpyAsync(b->d_pair_expert, b->h_u32, n_pairs * 4, cudaMemcpyHostToDevice, b->compute));
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(weights)",
     cudaMemcpyAsync(b->d_pair_weight, b->h_f32, n_pairs * 4, cudaMemcpyHostToDevice, b->compute));
  CU(MER_ERR_SUBMISSION, "cudaMemsetAsync(status)", cudaMemsetAsync(b->d_status, 0, 4, b->compute));
  d.n_groups = single_group ? 1u : (uint32_t)n_pairs;
  d.max_group_tokens = single_group ? (uint32_t)n_pairs : 1u;
  d.active_groups_hint = d.n_groups;
  bind_ffn(b, d);
  CU(MER_ERR_SUBMISSION, "wait for uploads", order_after_copies(b, b->compute));
  CU(MER_ERR_SUBMISSION, "group kernel", launch_groups_from_pairs(d, b->compute, launches));
  d.fuse_combine = combine_follows ? 1 : 0;
  CU(MER_ERR_SUBMISSION, "expert FFN kernels", run_ffn(b, d, b->compute, launches));
  if (!combine_follows) CU(MER_ERR_SUBMISSION, "partial-sum kernel", launch_reduce_parts(d, b->compute, launches));
  return MER_OK;
}

int finish_host_call(mer_backend *b, uint32_t layer, uint32_t expert, int launches, size_t n_experts_run) {
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(status)",
     cudaMemcpyAsync(b->h_u32 + b->max_pairs, b->d_status, 4, cudaMemcpyDeviceToHost, b->compute));
  CU(MER_ERR_READBACK_MAP, "cudaStreamSynchronize", cudaStreamSynchronize(b->compute));
  b->ctr.kernel_launches += (uint64_t)launches;
  b->ctr.gpu_dispatch_attempts += n_experts_run;
  int rc = check_device_status(b, b->h_u32[b->max_pairs], layer, expert);
  if (rc && rc != MER_ERR_NUMERICAL) {
    b->ctr.gpu_dispatch_failures += n_experts_run;  // counted once, never replayed (engine.rs:6624-6642)
    return rc;
  }
  b->ctr.gpu_dispatch_successes += n_experts_run;
  return rc;
}

}  // namespace

// ------------------------------------------------------------------------------- exports

MER_EXPORT int mer_abi_version(void) { return MER_ABI_VERSION; }

MER_EXPORT const char *mer_error_kind_name(int kind) {
  switch (kind) {
    case MER_OK: return "ok";
    case MER_ERR_RESIDENCY_MISS: return "residency-miss";
    case MER_ERR_PHYSICAL_CAPACITY: return "physical-capacity";
    case MER_ERR_UPLOAD: return "upload";
    case MER_ERR_VALIDATION_DISPATCH: return "validation-dispatch";
    case MER_ERR_SUBMISSION: return "submission";
    case MER_ERR_READBACK_CHANNEL: return "readback-channel";
    case MER_ERR_READBACK_MAP: return "readback-map";
    case MER_ERR_DEVICE_LOST: return "device-lost";
    case MER_ERR_RUNTIME_INVARIANT: return "runtime-invariant";
    case MER_ERR_INELIGIBLE: return "ineligible";
    case MER_ERR_TIMEOUT: return "timeout";
    case MER_ERR_INVALID_ARGUMENT: return "invalid-argument";
    case MER_ERR_NUMERICAL: return "numerical";
    default: return "unknown";
  }
}

MER_EXPORT uint64_t mer_expert_bytes(int32_t dtype, uint64_t d_model, uint64_t d_ff) {
  if (dtype != MER_DTYPE_Q4_0 && dtype != MER_DTYPE_Q8_0) return 0;
  uint64_t one = d_model * d_ff;
  return (one + 31) / 32 * block_bytes(dtype) * 3;
}

MER_EXPORT int mer_routed_expert_compatibility(int32_t dtype, uint64_t d_model, uint64_t d_ff) {
  // MAX_EXPERT_D_FF workspace bound and %32 alignment, backend/mod.rs:4691-4720; unaligned
  // shapes stay eligible here through the generic kernels.
  if (dtype != MER_DTYPE_Q4_0 && dtype != MER_DTYPE_Q8_0) return MER_ERR_VALIDATION_DISPATCH;
  if (d_model == 0 || d_ff == 0 || d_model > MAX_DIM || d_ff > MAX_DIM) return MER_ERR_VALIDATION_DISPATCH;
  return MER_OK;
}

MER_EXPORT int mer_backend_create(const mer_backend_cfg *cfg, mer_backend **out) {
  if (!cfg || !out) return MER_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  if (mer_routed_expert_compatibility(cfg->dtype, cfg->d_model, cfg->d_ff) != MER_OK) return MER_ERR_VALIDATION_DISPATCH;
  if (cfg->max_experts == 0 || cfg->max_tokens == 0 || cfg->max_top_k == 0 || cfg->max_top_k > 32) return MER_ERR_INVALID_ARGUMENT;
  int n_dev = 0;
  if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
    cudaGetLastError();
    return MER_ERR_DEVICE_LOST;  // no CPU fallback: without a CUDA device nothing can run
  }
  if (cfg->device < 0 || cfg->device >= n_dev) return MER_ERR_INVALID_ARGUMENT;
  mer_backend *b = new (std::nothrow) mer_backend();
  if (!b) return MER_ERR_PHYSICAL_CAPACITY;
  b->cfg = *cfg;
  const uint32_t layer = 0, expert = MER_NONE;
  (void)layer, (void)expert;
  auto bail = [&](int rc) {
    free_all(b);
    delete b;
    return rc;
  };
#define CB(call)                                   \
  do {                                             \
    if ((call) != cudaSuccess) {                   \
      cudaGetLastError();                          \
      return bail(MER_ERR_PHYSICAL_CAPACITY);      \
    }                                              \
  } while (0)
  CB(cudaSetDevice(cfg->device));
  cudaDeviceProp prop{};
  CB(cudaGetDeviceProperties(&prop, cfg->device));
  b->sm_count = prop.multiProcessorCount;
  b->expert_bytes = (size_t)mer_expert_bytes(cfg->dtype, cfg->d_model, cfg->d_ff);
  b->slot_stride = (SLOT_HEADER_BYTES + b->expert_bytes + SLOT_ALIGN - 1) / SLOT_ALIGN * SLOT_ALIGN;
  b->n_slots = (size_t)(cfg->vram_capacity_bytes / b->slot_stride);
  if (b->n_slots == 0) return bail(MER_ERR_PHYSICAL_CAPACITY);
  if (b->n_slots > cfg->max_experts) b->n_slots = cfg->max_experts;
  b->slots.resize(b->n_slots);
  CB(cudaStreamCreateWithFlags(&b->compute, cudaStreamNonBlocking));
  CB(cudaStreamCreateWithFlags(&b->copy, cudaStreamNonBlocking));
  CB(cudaEventCreateWithFlags(&b->ev_compute_done, cudaEventDisableTiming));
  CB(cudaEventCreateWithFlags(&b->ev_copy_done, cudaEventDisableTiming));
  for (auto &e : b->ev_stage) CB(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  CB(cudaMalloc((void **)&b->arena, b->n_slots * b->slot_stride));
  CB(cudaMalloc((void **)&b->d_expert_ptr, sizeof(void *) * cfg->max_experts));
  CB(cudaMemset((void *)b->d_expert_ptr, 0, sizeof(void *) * cfg->max_experts));
  CB(cudaHostAlloc((void **)&b->h_expert_ptr, sizeof(void *) * cfg->max_experts, cudaHostAllocDefault));
  memset((void *)b->h_expert_ptr, 0, sizeof(void *) * cfg->max_experts);
  CB(cudaHostAlloc((void **)&b->h_stage[0], STAGE_BYTES, cudaHostAllocDefault));
  CB(cudaHostAlloc((void **)&b->h_stage[1], STAGE_BYTES, cudaHostAllocDefault));
  CB(cudaHostAlloc((void **)&b->h_hdr, sizeof(SlotHeader) * b->n_slots, cudaHostAllocDefault));
  const size_t D = cfg->d_model, F = cfg->d_ff, T = cfg->max_tokens;
  b->max_pairs = cfg->max_tokens * cfg->max_top_k;
  const size_t P = b->max_pairs;
  b->max_groups = (uint32_t)std::max<size_t>(P, 4096) + 2;
  b->max_router_experts = 4096;
  CB(cudaMalloc((void **)&b->d_x, T * D * 4));
  CB(cudaMalloc((void **)&b->d_out, T * D * 4));
  CB(cudaMalloc((void **)&b->d_h, P * F * 4));
  CB(cudaMalloc((void **)&b->d_y, P * D * 4));
  CB(cudaMalloc((void **)&b->d_pair_weight, P * 4));
  CB(cudaMalloc((void **)&b->d_pair_expert, P * 4));
  CB(cudaMalloc((void **)&b->d_group_expert, (size_t)b->max_groups * 4));
  CB(cudaMalloc((void **)&b->d_offsets, ((size_t)b->max_groups + 1) * 4));
  CB(cudaMalloc((void **)&b->d_group_count, (size_t)b->max_groups * 2 * 4));
  CB(cudaMemset(b->d_group_count, 0, (size_t)b->max_groups * 2 * 4));
  CB(cudaMalloc((void **)&b->d_perm, P * 4));
  CB(cudaMalloc((void **)&b->d_logits, T * b->max_router_experts * 4));
  CB(cudaMalloc((void **)&b->d_status, 4));
  CB(cudaMalloc((void **)&b->d_counters, (T + 1) * 4));
  CB(cudaMemset(b->d_status, 0, 4));
  CB(cudaMemset(b->d_counters, 0, (T + 1) * 4));
  CB(cudaMalloc((void **)&b->d_f16, std::max(P, T) * D * 2));
  CB(cudaHostAlloc((void **)&b->h_u32, (P + 1) * 4, cudaHostAllocDefault));
  CB(cudaHostAlloc((void **)&b->h_f32, P * 4, cudaHostAllocDefault));
  if (stream_ffn_supported(cfg->dtype, (uint32_t)D, (uint32_t)F)) {
    b->packed = true;
    CB(cudaMalloc((void **)&b->d_raw_stage, b->expert_bytes));
    size_t sb = stream_ffn_scratch_bytes((uint32_t)P, (uint32_t)D, (uint32_t)F);
    if (sb) {
      CB(cudaMalloc(&b->d_stream_scratch, sb));
      CB(cudaMemset(b->d_stream_scratch, 0, sb));
    }
    if (sb && T >= 12 && gemm_ffn_supported(cfg->dtype, (uint32_t)D, (uint32_t)F)) {
      // token rows of a dispatch may be (token, slot) pairs of other ranks (NCCL all-to-all mode): size per-row scratch by pairs
      b->gemm_scratch_bytes = gemm_ffn_scratch_bytes((uint32_t)std::max(T, P), (uint32_t)P, (uint32_t)D, (uint32_t)F);
      CB(cudaMalloc(&b->d_gemm_scratch, b->gemm_scratch_bytes));
    }
  }
  CB(cudaDeviceSynchronize());
#undef CB
  b->ctr.arena_bytes = b->n_slots * b->slot_stride;
  b->ctr.slot_stride_bytes = b->slot_stride;
  b->ctr.slot_count = b->n_slots;
  *out = b;
  return MER_OK;
}

MER_EXPORT void mer_backend_destroy(mer_backend *b) {
  if (!b) return;
  cudaSetDevice(b->cfg.device);
  cudaDeviceSynchronize();
  free_all(b);
  delete b;
}

MER_EXPORT int mer_backend_synchronize(mer_backend *b) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = MER_NONE;
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  CU(MER_ERR_UPLOAD, "cudaStreamSynchronize(copy)", cudaStreamSynchronize(b->copy));
  CU(MER_ERR_READBACK_MAP, "cudaStreamSynchronize(compute)", cudaStreamSynchronize(b->compute));
  return MER_OK;
}

MER_EXPORT int mer_expert_admit(mer_backend *b, uint32_t expert_id, uint64_t generation, const void *host_blob, size_t bytes,
                                uint32_t flags) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  return admit_impl(b, expert_id, generation, host_blob, bytes, flags, false);
}

MER_EXPORT int mer_expert_admit_device(mer_backend *b, uint32_t expert_id, uint64_t generation, const void *device_blob,
                                       size_t bytes, uint32_t flags) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  return admit_impl(b, expert_id, generation, device_blob, bytes, flags, true);
}

MER_EXPORT int mer_expert_admit_file(mer_backend *b, uint32_t expert_id, uint64_t generation, const char *path, size_t block_align,
                                     uint32_t flags) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = expert_id;
  if (!path) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null path");
  FILE *f = fopen(path, "rb");
  if (!f) return fail(b, MER_ERR_UPLOAD, layer, expert, "cannot open %s", path);
  struct Closer {
    FILE *f;
    ~Closer() { fclose(f); }
  } closer{f};
  if (fseeko(f, 0, SEEK_END) != 0) return fail(b, MER_ERR_UPLOAD, layer, expert, "cannot seek in %s", path);
  const uint64_t file_bytes = (uint64_t)ftello(f);
  // the header region: at most one block (a UTH header is padded to block_align)
  std::vector<uint8_t> head(std::min<uint64_t>(file_bytes, std::max<size_t>(block_align, 128)));
  if (fseeko(f, 0, SEEK_SET) != 0 || fread(head.data(), 1, head.size(), f) != head.size())
    return fail(b, MER_ERR_UPLOAD, layer, expert, "cannot read the header region of %s", path);
  mer_uth_info h{};
  mer_uth_probe_prefix(head.data(), head.size(), file_bytes, block_align, &h);
  uint64_t payload_off = 0;
  uint64_t range_off[3], range_len[3];
  const uint64_t proj = b->expert_bytes / 3;
  if (h.kind == MER_UTH_KIND_NONE) {
    // a legacy blob: the file is the payload (plus page padding)
    for (int i = 0; i < 3; i++) range_off[i] = i * proj, range_len[i] = proj;
  } else {
    if (h.dtype != b->cfg.dtype)
      return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "%s holds dtype id %u, the backend runs %s", path, h.uth_dtype_id,
                  b->cfg.dtype == MER_DTYPE_Q4_0 ? "q4_0" : "q8_0");
    if (h.d_model != b->cfg.d_model || h.d_ff != b->cfg.d_ff)
      return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "%s is %llux%llu, the backend %llux%llu", path, (unsigned long long)h.d_model,
                  (unsigned long long)h.d_ff, (unsigned long long)b->cfg.d_model, (unsigned long long)b->cfg.d_ff);
    payload_off = h.payload_offset;
    if (h.kind == MER_UTH_KIND_UTH2) {
      // the probe saw only the header region: validate the ranges against the real payload length
      const uint64_t payload_len = file_bytes > payload_off ? file_bytes - payload_off : 0;
      for (int i = 0; i < 3; i++) {
        range_off[i] = h.proj[i].offset, range_len[i] = h.proj[i].len;
        if (range_len[i] != proj || range_off[i] + range_len[i] > payload_len)
          return fail(b, MER_ERR_UPLOAD, layer, expert, "%s: projection %d covers %llu bytes at %llu, need %llu inside %llu", path, i,
                      (unsigned long long)range_len[i], (unsigned long long)range_off[i], (unsigned long long)proj,
                      (unsigned long long)payload_len);
      }
    } else {
      for (int i = 0; i < 3; i++) range_off[i] = i * proj, range_len[i] = proj;
    }
  }
  uint64_t need = 0;
  for (int i = 0; i < 3; i++) need = std::max(need, payload_off + range_off[i] + range_len[i]);
  if (file_bytes < need)
    return fail(b, MER_ERR_UPLOAD, layer, expert, "%s has %llu bytes, the expert needs %llu", path, (unsigned long long)file_bytes,
                (unsigned long long)need);
  ChunkReader reader = [&](size_t off, size_t n, uint8_t *dst) -> bool {
    while (n) {  // canonical offset -> (projection, offset inside it) -> file offset
      const size_t pi = off / proj, in = off % proj, take = std::min<size_t>(n, proj - in);
      if (pi >= 3 || fseeko(f, (off_t)(payload_off + range_off[pi] + in), SEEK_SET) != 0 || fread(dst, 1, take, f) != take) return false;
      off += take, dst += take, n -= take;
    }
    return true;
  };
  return admit_impl(b, expert_id, generation, head.data(), b->expert_bytes, flags, false, &reader);  // the file is read completely before this returns
}

MER_EXPORT int mer_expert_retire(mer_backend *b, uint32_t expert_id, uint64_t generation) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = expert_id;
  std::lock_guard<std::mutex> lock(b->mu);
  auto it = b->id2slot.find(expert_id);
  if (it == b->id2slot.end() || b->slots[it->second].generation != generation) return MER_OK;  // not current: nothing to retire
  CU(MER_ERR_UPLOAD, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  CU(MER_ERR_UPLOAD, "order the copy stream after the readers", copy_waits_for_readers(b));
  b->h_expert_ptr[expert_id] = nullptr;
  CU(MER_ERR_UPLOAD, "cudaMemcpyAsync(table)",
     cudaMemcpyAsync((void *)(b->d_expert_ptr + expert_id), (void *)(b->h_expert_ptr + expert_id), sizeof(void *),
                     cudaMemcpyHostToDevice, b->copy));
  CU(MER_ERR_UPLOAD, "cudaEventRecord(copy)", cudaEventRecord(b->ev_copy_done, b->copy));
  b->copy_pending = true;
  b->slots[it->second] = Slot{};
  b->id2slot.erase(it);
  return MER_OK;
}

MER_EXPORT int mer_expert_contains_generation(mer_backend *b, uint32_t expert_id, uint64_t generation) {
  if (!b) return 0;
  std::lock_guard<std::mutex> lock(b->mu);
  auto it = b->id2slot.find(expert_id);
  return it != b->id2slot.end() && b->slots[it->second].generation == generation;
}

// ---- the logical tier (vram_tier.cpp) driving the physical slots
namespace {
// Frees the physical slot of `id` whatever generation it holds (the policy evicted the id).  Caller holds b->mu.
int retire_physical_locked(mer_backend *b, uint32_t id, uint32_t flags) {
  const uint32_t layer = 0, expert = id;
  auto it = b->id2slot.find(id);
  if (it == b->id2slot.end()) return MER_OK;
  CU(MER_ERR_UPLOAD, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  if (!(flags & MER_ADMIT_NO_READER_WAIT)) CU(MER_ERR_UPLOAD, "order the copy stream after the readers", copy_waits_for_readers(b));
  b->h_expert_ptr[id] = nullptr;
  CU(MER_ERR_UPLOAD, "cudaMemcpyAsync(table)",
     cudaMemcpyAsync((void *)(b->d_expert_ptr + id), (void *)(b->h_expert_ptr + id), sizeof(void *), cudaMemcpyHostToDevice, b->copy));
  CU(MER_ERR_UPLOAD, "cudaEventRecord(copy)", cudaEventRecord(b->ev_copy_done, b->copy));
  b->copy_pending = true;
  b->slots[it->second] = Slot{};
  b->id2slot.erase(it);
  b->ctr.evictions++;
  return MER_OK;
}

int retire_evicted(mer_backend *b, const uint32_t *ids, size_t n, uint32_t flags) {
  std::lock_guard<std::mutex> lock(b->mu);
  for (size_t i = 0; i < n; i++) {
    int rc = retire_physical_locked(b, ids[i], flags);
    if (rc) return rc;
  }
  return MER_OK;
}

bool physical_has(mer_backend *b, uint32_t id, uint64_t generation) {
  std::lock_guard<std::mutex> lock(b->mu);
  auto it = b->id2slot.find(id);
  return it != b->id2slot.end() && b->slots[it->second].generation == generation;
}
}  // namespace

MER_EXPORT int mer_expert_demand_admit(mer_backend *b, mer_gpu_cache *cache, uint32_t expert_id, const void *host_blob, size_t bytes,
                                       uint32_t flags, uint64_t *generation) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = expert_id;
  if (!cache) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null cache");
  if (expert_id >= b->cfg.max_experts)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "expert id %u outside the id space of %u", expert_id, b->cfg.max_experts);
  if (host_blob && bytes < b->expert_bytes)
    return fail(b, MER_ERR_UPLOAD, layer, expert, "blob has %zu bytes, need %zu", bytes, b->expert_bytes);
  // The policy accounts the logical payload (the bytes a slot holds), not the caller's page padding.
  const uint64_t logical = b->expert_bytes;
  const int pre = mer_gpu_cache_demand_admission_preflight(cache, expert_id, logical);
  if (pre == MER_DEMAND_ERR_EXCEEDS_LRU_CAPACITY)
    return fail(b, MER_ERR_PHYSICAL_CAPACITY, layer, expert, "expert payload of %llu bytes exceeds the logical LRU capacity",
                (unsigned long long)logical);
  if (pre < 0) return fail(b, MER_ERR_UPLOAD, layer, expert, "empty expert payload");
  mer_gpu_admission adm{};
  if (pre == MER_DEMAND_ALREADY_ADMITTED) {
    if (!mer_gpu_cache_current_admission(cache, expert_id, &adm))
      return fail(b, MER_ERR_RESIDENCY_MISS, layer, expert, "the admission vanished between the preflight and the lookup");
    if (generation) *generation = adm.generation;
    if (physical_has(b, expert_id, adm.generation)) return MER_OK;
    // admitted logically, no physical copy of that generation yet: the lazy upload of backend/mod.rs:3916-3990
    if (!host_blob) return fail(b, MER_ERR_RESIDENCY_MISS, layer, expert, "admitted logically but not uploaded, and no payload was passed");
    return admit_impl(b, expert_id, adm.generation, host_blob, bytes, flags | (adm.region == MER_REGION_ANCHOR ? MER_ADMIT_ANCHOR : 0u), false);
  }
  if (!host_blob) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "a new admission needs the expert payload");
  uint32_t evicted[64];
  size_t n_ev = 0;
  uint64_t gen = 0;
  const int rc = mer_gpu_cache_demand_admit_lru(cache, expert_id, logical, (uint64_t)(uintptr_t)host_blob, evicted, 64, &n_ev, &gen);
  if (rc == MER_DEMAND_ERR_GENERATION_EXHAUSTED)
    return fail(b, MER_ERR_RUNTIME_INVARIANT, layer, expert, "logical GPU admission generation space exhausted");
  if (rc == MER_DEMAND_ERR_EXCEEDS_LRU_CAPACITY)
    return fail(b, MER_ERR_PHYSICAL_CAPACITY, layer, expert, "expert payload exceeds the logical LRU capacity");
  if (rc < 0) return fail(b, MER_ERR_UPLOAD, layer, expert, "empty expert payload");
  if (rc == MER_DEMAND_ALREADY_ADMITTED) {  // another thread admitted it after the preflight: use that admission
    mer_gpu_cache_current_admission(cache, expert_id, &adm);
    gen = adm.generation;
  }
  if (generation) *generation = gen;
  if (n_ev > 64)
    return fail(b, MER_ERR_RUNTIME_INVARIANT, layer, expert, "one admission evicted %zu experts, more than this call can retire", n_ev);
  int rr = retire_evicted(b, evicted, n_ev, flags);
  if (rr) return rr;
  if (physical_has(b, expert_id, gen)) return MER_OK;
  return admit_impl(b, expert_id, gen, host_blob, bytes, flags & ~MER_ADMIT_ANCHOR, false);
}

MER_EXPORT int mer_expert_hot_promote(mer_backend *b, mer_gpu_cache *cache, uint32_t expert_id, const void *host_blob, size_t bytes,
                                      uint32_t flags, int *outcome) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = expert_id;
  if (!cache || !outcome) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null cache or outcome");
  if (expert_id >= b->cfg.max_experts)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "expert id %u outside the id space of %u", expert_id, b->cfg.max_experts);
  int o = mer_gpu_cache_promote_hot_existing(cache, expert_id);
  uint32_t evicted[64];
  size_t n_ev = 0;
  uint64_t gen = 0;
  if (o == MER_HOT_PAYLOAD_REQUIRED && host_blob) {
    if (bytes < b->expert_bytes) {
      mer_gpu_cache_cancel_promotion(cache, expert_id);
      return fail(b, MER_ERR_UPLOAD, layer, expert, "blob has %zu bytes, need %zu", bytes, b->expert_bytes);
    }
    o = mer_gpu_cache_promote_hot_sync(cache, expert_id, b->expert_bytes, (uint64_t)(uintptr_t)host_blob, evicted, 64, &n_ev, &gen);
  }
  *outcome = o;
  if (n_ev > 64) return fail(b, MER_ERR_RUNTIME_INVARIANT, layer, expert, "one promotion evicted %zu experts", n_ev);
  int rr = retire_evicted(b, evicted, n_ev, flags);
  if (rr) return rr;
  mer_gpu_admission adm{};
  if (!mer_gpu_cache_current_admission(cache, expert_id, &adm)) return MER_OK;  // nothing admitted (payload required, no capacity ...)
  const bool anchor = adm.region == MER_REGION_ANCHOR;
  if (physical_has(b, expert_id, adm.generation)) {
    std::lock_guard<std::mutex> lock(b->mu);
    auto it = b->id2slot.find(expert_id);
    if (it != b->id2slot.end()) b->slots[it->second].anchor = anchor;
    return MER_OK;
  }
  if (!host_blob) return MER_OK;  // the physical upload stays lazy: the next demand for the id brings the payload
  return admit_impl(b, expert_id, adm.generation, host_blob, bytes, (flags & ~MER_ADMIT_ANCHOR) | (anchor ? MER_ADMIT_ANCHOR : 0u), false);
}

MER_EXPORT int mer_expert_touch(mer_backend *b, mer_gpu_cache *cache, const uint32_t *expert_ids, size_t n) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  if (!expert_ids && n) return fail(b, MER_ERR_INVALID_ARGUMENT, 0, MER_NONE, "null ids");
  for (size_t i = 0; i < n; i++) {
    if (expert_ids[i] == MER_NONE) continue;
    if (cache) (void)mer_gpu_cache_get(cache, expert_ids[i], nullptr);
  }
  std::lock_guard<std::mutex> lock(b->mu);
  for (size_t i = 0; i < n; i++) {
    auto it = b->id2slot.find(expert_ids[i]);
    if (it != b->id2slot.end()) b->slots[it->second].last_use = ++b->tick;
  }
  return MER_OK;
}

MER_EXPORT int mer_router_install(mer_backend *b, uint32_t layer, const float *host_weights, const mer_router_cfg *cfg) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  if (!host_weights || !cfg) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null router weights or cfg");
  // LinearGate::new asserts (gating.rs:149-158)
  if (cfg->top_k == 0 || cfg->top_k > cfg->num_experts)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "top_k must be in 1..=num_experts");
  uint32_t slots = cfg->top_k + (cfg->shared_expert_id != MER_NONE ? 1u : 0u);
  if (slots > b->cfg.max_top_k || cfg->top_k > 32)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "top_k %u (+shared) exceeds max_top_k %u", cfg->top_k, b->cfg.max_top_k);
  if (cfg->num_experts > b->max_router_experts || (uint64_t)(layer + 1) * cfg->num_experts > b->cfg.max_experts)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "layer %u x %u experts exceeds the id space of %u", layer,
                cfg->num_experts, b->cfg.max_experts);
  if (cfg->n_group > 64) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "n_group %u > 64", cfg->n_group);
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_UPLOAD, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  RouterEntry &r = b->routers[layer];
  CU(MER_ERR_UPLOAD, "cudaStreamSynchronize", cudaStreamSynchronize(b->compute));
  drop_graphs(b);
  if (r.d_w) cudaFree(r.d_w), r.d_w = nullptr;
  if (r.d_cbias) cudaFree(r.d_cbias), r.d_cbias = nullptr;
  if (r.d_lbias) cudaFree(r.d_lbias), r.d_lbias = nullptr;
  size_t wbytes = (size_t)cfg->num_experts * b->cfg.d_model * 4, ebytes = (size_t)cfg->num_experts * 4;
  CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(router)", cudaMalloc((void **)&r.d_w, wbytes));
  CU(MER_ERR_UPLOAD, "cudaMemcpy(router)", cudaMemcpy(r.d_w, host_weights, wbytes, cudaMemcpyHostToDevice));
  if (cfg->correction_bias) {
    CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(bias)", cudaMalloc((void **)&r.d_cbias, ebytes));
    CU(MER_ERR_UPLOAD, "cudaMemcpy(bias)", cudaMemcpy(r.d_cbias, cfg->correction_bias, ebytes, cudaMemcpyHostToDevice));
  }
  if (cfg->logit_bias) {
    CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(bias)", cudaMalloc((void **)&r.d_lbias, ebytes));
    CU(MER_ERR_UPLOAD, "cudaMemcpy(bias)", cudaMemcpy(r.d_lbias, cfg->logit_bias, ebytes, cudaMemcpyHostToDevice));
  }
  r.dev.w = r.d_w;
  r.dev.correction_bias = r.d_cbias;
  r.dev.logit_bias = r.d_lbias;
  r.dev.num_experts = cfg->num_experts;
  r.dev.top_k = cfg->top_k;
  r.dev.scoring = cfg->scoring_func;
  r.dev.normalise = cfg->normalise_topk;
  r.dev.n_group = cfg->n_group < 1 ? 1 : cfg->n_group;  // with_routing: n_group.max(1), gating.rs:234
  r.dev.topk_group = cfg->topk_group;
  r.dev.scaling = cfg->routed_scaling_factor;
  r.dev.shared_expert_id = cfg->shared_expert_id;
  r.dev.id_base = layer * cfg->num_experts;
  return MER_OK;
}

MER_EXPORT int mer_layer_install(mer_backend *b, uint32_t layer, const mer_layer_cfg *cfg) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  if (!cfg) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null layer cfg");
  if (cfg->rms_weight && !(cfg->rms_eps >= 0.0f)) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "rms_eps must be >= 0");
  std::lock_guard<std::mutex> lock(b->mu);
  auto it = b->routers.find(layer);
  if (it == b->routers.end()) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "install the layer's router first (layer %u)", layer);
  CU(MER_ERR_UPLOAD, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  CU(MER_ERR_UPLOAD, "cudaStreamSynchronize", cudaStreamSynchronize(b->compute));
  drop_graphs(b);
  RouterEntry &r = it->second;
  const size_t D = b->cfg.d_model;
  if (r.d_rms_w) cudaFree(r.d_rms_w), r.d_rms_w = nullptr;
  if (r.d_shared_gate) cudaFree(r.d_shared_gate), r.d_shared_gate = nullptr;
  if (cfg->rms_weight) {
    CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(rms weight)", cudaMalloc((void **)&r.d_rms_w, D * 4));
    CU(MER_ERR_UPLOAD, "cudaMemcpy(rms weight)", cudaMemcpy(r.d_rms_w, cfg->rms_weight, D * 4, cudaMemcpyHostToDevice));
    if (!b->d_xn) CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(normed rows)", cudaMalloc((void **)&b->d_xn, (size_t)b->cfg.max_tokens * D * 4));
  }
  if (cfg->shared_gate) {
    CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(shared gate)", cudaMalloc((void **)&r.d_shared_gate, D * 4));
    CU(MER_ERR_UPLOAD, "cudaMemcpy(shared gate)", cudaMemcpy(r.d_shared_gate, cfg->shared_gate, D * 4, cudaMemcpyHostToDevice));
    if (!b->d_shared_scale)
      CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(shared scale)", cudaMalloc((void **)&b->d_shared_scale, (size_t)b->cfg.max_tokens * 4));
  }
  r.rms_eps = cfg->rms_eps;
  r.layer_flags = cfg->flags;
  return MER_OK;
}

namespace {
// Enqueues router (+ optional FFN + combine) for device-resident x on stream s.
int enqueue_layer(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, float *d_out, bool run_ffn_too,
                  cudaStream_t s, int *launches, MoeDispatch *out_d, bool capturing = false) {
  const uint32_t expert = MER_NONE;
  auto it = b->routers.find(layer);
  if (it == b->routers.end()) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "no router installed for layer %u", layer);
  if (n_tokens == 0 || n_tokens > b->cfg.max_tokens)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "n_tokens %zu outside 1..=%u", n_tokens, b->cfg.max_tokens);
  const RouterDev &r = it->second.dev;
  MoeDispatch d = base_dispatch(b);
  d.n_tokens = (uint32_t)n_tokens;
  d.slots = r.top_k + (r.shared_expert_id != MER_NONE ? 1u : 0u);
  d.n_groups = r.num_experts + (r.shared_expert_id != MER_NONE ? 1u : 0u);
  d.max_group_tokens = d.n_tokens;  // a token reaches an expert at most once
  d.active_groups_hint = std::min(d.n_groups, d.n_tokens * d.slots);
  if (run_ffn_too) bind_ffn(b, d);
  d.x = d_x;
  d.out = d_out;
  CU(MER_ERR_SUBMISSION, "cudaMemsetAsync(status)", cudaMemsetAsync(b->d_status, 0, 4, s));
  if (!capturing) CU(MER_ERR_SUBMISSION, "wait for uploads", order_after_copies(b, s));
  cudaEvent_t *ev = (run_ffn_too && !capturing) ? next_timing_set(b) : nullptr;
  if (ev) cudaEventRecord(ev[0], s);
  // optional steps in front of the block: RMSNorm of the rows (router and experts then read the normed rows) and the
  // shared expert's gate scalar; behind it: the residual add in the combine
  RouterDev rl = r;
  const RouterEntry &re = it->second;
  if (re.d_rms_w || re.d_shared_gate) {
    const bool gated = re.d_shared_gate && r.shared_expert_id != MER_NONE;
    CU(MER_ERR_SUBMISSION, "pre-MoE kernel",
       launch_pre_moe(d_x, d.n_tokens, d.D, re.d_rms_w, re.rms_eps, gated ? re.d_shared_gate : nullptr, b->d_xn, b->d_shared_scale, s, launches));
    if (re.d_rms_w) d.x = b->d_xn;
    if (gated) rl.shared_scale = b->d_shared_scale;
  }
  if (re.layer_flags & MER_LAYER_RESIDUAL) d.residual = d_x, d.routed_slots = r.top_k;
  const RouterDev &r2 = rl;
  CU(MER_ERR_SUBMISSION, "router kernel", launch_router(r2, d, b->cfg.max_tokens, s, launches));
  if (run_ffn_too) {
    if (ev) cudaEventRecord(ev[1], s);
    d.fuse_combine = 1;
    CU(MER_ERR_SUBMISSION, "expert FFN kernels", run_ffn(b, d, s, launches, ev ? ev[2] : nullptr));
    if (ev) cudaEventRecord(ev[3], s);
    CU(MER_ERR_SUBMISSION, "combine kernel", launch_combine(d, s, launches));
    if (ev) cudaEventRecord(ev[4], s);
  }
  if (out_d) *out_d = d;
  return MER_OK;
}
}  // namespace

MER_EXPORT int mer_router_route(mer_backend *b, uint32_t layer, const float *x, size_t n_tokens, uint32_t *ids, float *weights) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  if (!x || !ids || !weights) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  if (n_tokens == 0 || n_tokens > b->cfg.max_tokens)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "n_tokens %zu outside 1..=%u", n_tokens, b->cfg.max_tokens);
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(x)",
     cudaMemcpyAsync(b->d_x, x, n_tokens * b->cfg.d_model * 4, cudaMemcpyHostToDevice, b->compute));
  int launches = 0;
  MoeDispatch d;
  int rc = enqueue_layer(b, layer, b->d_x, n_tokens, b->d_out, false, b->compute, &launches, &d);
  if (rc) return rc;
  const RouterDev &r = b->routers[layer].dev;
  // ids/weights on the device are [n_tokens x slots]; the caller gets the top_k routed columns with local ids
  size_t P = n_tokens * d.slots;
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(ids)", cudaMemcpyAsync(b->h_u32, b->d_pair_expert, P * 4, cudaMemcpyDeviceToHost, b->compute));
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(w)", cudaMemcpyAsync(b->h_f32, b->d_pair_weight, P * 4, cudaMemcpyDeviceToHost, b->compute));
  rc = finish_host_call(b, layer, expert, launches, 0);
  for (size_t t = 0; t < n_tokens; t++)
    for (uint32_t s = 0; s < r.top_k; s++) {
      uint32_t g = b->h_u32[t * d.slots + s];
      ids[t * r.top_k + s] = g == MER_NONE ? MER_NONE : g - r.id_base;
      weights[t * r.top_k + s] = b->h_f32[t * d.slots + s];
    }
  b->ctr.hidden_upload_bytes += n_tokens * b->cfg.d_model * 4;
  b->ctr.readback_bytes += P * 8;
  return rc;
}

MER_EXPORT int mer_routed_expert_matmul_batch(mer_backend *b, uint32_t layer, const uint32_t *expert_ids, size_t n,
                                              const uint16_t *x, size_t d_model, size_t d_ff, uint16_t *out) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  uint32_t expert = (expert_ids && n) ? expert_ids[0] : MER_NONE;
  if (!expert_ids || !x || !out) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  std::lock_guard<std::mutex> lock(b->mu);
  if (n == 0 || n > b->cfg.max_top_k || n > b->max_pairs)
    return fail(b, MER_ERR_INELIGIBLE, layer, expert, "batch of %zu experts is outside 1..=%u", n, b->cfg.max_top_k);
  int rc = validate_shape_args(b, layer, expert, d_model, d_ff);
  if (rc) return rc;
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  b->ctr.batch_calls += n > 1;
  b->ctr.selected_routed_experts += n;
  for (size_t i = 0; i < n; i++)
    if ((rc = require_resident(b, layer, expert_ids[i])) != MER_OK) {
      b->ctr.gpu_dispatch_attempts += n;
      b->ctr.gpu_dispatch_failures += n;
      return rc;
    }
  const size_t D = b->cfg.d_model;
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(x)", cudaMemcpyAsync(b->d_f16, x, D * 2, cudaMemcpyHostToDevice, b->compute));
  CU(MER_ERR_SUBMISSION, "f16->f32", launch_f16_to_f32(b->d_f16, b->d_x, D, b->compute));
  MoeDispatch d = base_dispatch(b);
  d.n_tokens = 1;
  d.slots = (uint32_t)n;
  d.x = b->d_x;
  d.out = b->d_out;
  int launches = 1;
  rc = dispatch_given_routing(b, layer, d, expert_ids, nullptr, n, false, &launches);
  if (rc) return rc;
  CU(MER_ERR_SUBMISSION, "f32->f16", launch_f32_to_f16(b->d_y, b->d_f16, n * D, b->compute));
  launches++;
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(out)", cudaMemcpyAsync(out, b->d_f16, n * D * 2, cudaMemcpyDeviceToHost, b->compute));
  b->ctr.hidden_upload_bytes += D * 2;
  b->ctr.readback_bytes += n * D * 2;
  return finish_host_call(b, layer, expert, launches, n);
}

MER_EXPORT int mer_routed_expert_matmul(mer_backend *b, uint32_t layer, uint32_t expert_id, const uint16_t *x, size_t d_model,
                                        size_t d_ff, uint16_t *out) {
  return mer_routed_expert_matmul_batch(b, layer, &expert_id, 1, x, d_model, d_ff, out);
}

MER_EXPORT int mer_routed_expert_forward_f32(mer_backend *b, uint32_t layer, uint32_t expert_id, const float *x, size_t n_tokens,
                                             float *out) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = expert_id;
  if (!x || !out) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  std::lock_guard<std::mutex> lock(b->mu);
  if (n_tokens == 0 || n_tokens > b->cfg.max_tokens || n_tokens > b->max_pairs)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "n_tokens %zu outside 1..=%u", n_tokens, b->cfg.max_tokens);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  b->ctr.selected_routed_experts += 1;
  int rc = require_resident(b, layer, expert_id);
  if (rc) {
    b->ctr.gpu_dispatch_attempts++, b->ctr.gpu_dispatch_failures++;
    return rc;
  }
  const size_t D = b->cfg.d_model;
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(x)", cudaMemcpyAsync(b->d_x, x, n_tokens * D * 4, cudaMemcpyHostToDevice, b->compute));
  MoeDispatch d = base_dispatch(b);
  d.n_tokens = (uint32_t)n_tokens;
  d.slots = 1;
  d.x = b->d_x;
  d.out = b->d_out;
  std::vector<uint32_t> ids(n_tokens, expert_id);
  int launches = 0;
  rc = dispatch_given_routing(b, layer, d, ids.data(), nullptr, n_tokens, true, &launches);
  if (rc) return rc;
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(out)", cudaMemcpyAsync(out, b->d_y, n_tokens * D * 4, cudaMemcpyDeviceToHost, b->compute));
  b->ctr.hidden_upload_bytes += n_tokens * D * 4;
  b->ctr.readback_bytes += n_tokens * D * 4;
  return finish_host_call(b, layer, expert, launches, 1);
}

MER_EXPORT int mer_moe_step_weighted_into(mer_backend *b, uint32_t layer, const float *x, const uint32_t *expert_ids,
                                          const float *weights, size_t n_slots, float *out) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  uint32_t expert = (expert_ids && n_slots) ? expert_ids[0] : MER_NONE;
  if (!x || !expert_ids || !weights || !out) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  std::lock_guard<std::mutex> lock(b->mu);
  if (n_slots == 0 || n_slots > b->cfg.max_top_k)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "n_slots %zu outside 1..=%u", n_slots, b->cfg.max_top_k);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  b->ctr.selected_routed_experts += n_slots;
  int rc;
  for (size_t i = 0; i < n_slots; i++)
    if ((rc = require_resident(b, layer, expert_ids[i])) != MER_OK) {
      b->ctr.gpu_dispatch_attempts += n_slots, b->ctr.gpu_dispatch_failures += n_slots;
      return rc;
    }
  const size_t D = b->cfg.d_model;
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(x)", cudaMemcpyAsync(b->d_x, x, D * 4, cudaMemcpyHostToDevice, b->compute));
  MoeDispatch d = base_dispatch(b);
  d.n_tokens = 1;
  d.slots = (uint32_t)n_slots;
  d.x = b->d_x;
  d.out = b->d_out;
  int launches = 0;
  rc = dispatch_given_routing(b, layer, d, expert_ids, weights, n_slots, false, &launches, true);
  if (rc) return rc;
  CU(MER_ERR_SUBMISSION, "combine kernel", launch_combine(d, b->compute, &launches));
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(out)", cudaMemcpyAsync(out, b->d_out, D * 4, cudaMemcpyDeviceToHost, b->compute));
  b->ctr.batch_calls += 1;
  b->ctr.hidden_upload_bytes += D * 4;
  b->ctr.readback_bytes += D * 4;
  return finish_host_call(b, layer, expert, launches, n_slots);
}

MER_EXPORT int mer_moe_layer_forward(mer_backend *b, uint32_t layer, const float *x, size_t n_tokens, float *out, uint32_t *ids,
                                     float *weights) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  if (!x || !out) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  if (n_tokens == 0 || n_tokens > b->cfg.max_tokens)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "n_tokens %zu outside 1..=%u", n_tokens, b->cfg.max_tokens);
  const size_t D = b->cfg.d_model;
  // Pinned host buffers and no routing wanted back: upload, layer, read-back and the status word are captured once
  // per (layer, n_tokens, x, out) and replayed as one graph launch (the call stays synchronous).
  if (!ids && !weights && b->graphs_ok && !b->timing_on && !(b->cfg.flags & MER_FLAG_NO_GRAPHS) && b->routers.count(layer)) {
    cudaPointerAttributes ax{}, ao{};
    const bool pinned = cudaPointerGetAttributes(&ax, x) == cudaSuccess && ax.type == cudaMemoryTypeHost &&
                        cudaPointerGetAttributes(&ao, out) == cudaSuccess && ao.type == cudaMemoryTypeHost;
    cudaGetLastError();
    if (pinned) {
      cudaStream_t s = b->compute;
      const void *host_tag = reinterpret_cast<const void *>(uintptr_t(1));  // marks host-entry graphs in the cache
      CU(MER_ERR_SUBMISSION, "wait for uploads", order_after_copies(b, s));
      mer_backend::GraphEntry *hit = nullptr;
      for (auto &g : b->graphs)
        if (g.layer == layer && g.n_tokens == n_tokens && g.x == x && g.out == out && g.ids == host_tag && g.stream == s) hit = &g;
      if (!hit) {
        if (b->graphs.size() >= 256) drop_graphs(b);
        cudaGraph_t graph = nullptr;
        cudaGraphExec_t exec = nullptr;
        int launches = 0, rc = MER_OK;
        bool ok = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        if (ok) {
          ok = cudaMemcpyAsync(b->d_x, x, n_tokens * D * 4, cudaMemcpyHostToDevice, s) == cudaSuccess;
          MoeDispatch d;
          if (ok) rc = enqueue_layer(b, layer, b->d_x, n_tokens, b->d_out, true, s, &launches, &d, true);
          if (ok && rc == MER_OK) ok = cudaMemcpyAsync(out, b->d_out, n_tokens * D * 4, cudaMemcpyDeviceToHost, s) == cudaSuccess;
          if (ok && rc == MER_OK)
            ok = cudaMemcpyAsync(b->h_u32 + b->max_pairs, b->d_status, 4, cudaMemcpyDeviceToHost, s) == cudaSuccess;
          cudaError_t ce = cudaStreamEndCapture(s, &graph);
          ok = ok && ce == cudaSuccess && graph != nullptr;
        }
        if (rc != MER_OK) {
          if (graph) cudaGraphDestroy(graph);
          cudaGetLastError();
          return rc;
        }
        if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
        if (graph) cudaGraphDestroy(graph);
        if (ok) {
          b->graphs.push_back({layer, n_tokens, x, out, host_tag, nullptr, s, exec, launches});
          hit = &b->graphs.back();
        } else {
          cudaGetLastError();
          b->graphs_ok = false;  // capture is not available here: plain launches from now on
        }
      }
      if (hit) {
        const RouterDev &r = b->routers[layer].dev;
        const size_t P = n_tokens * (r.top_k + (r.shared_expert_id != MER_NONE ? 1u : 0u));
        CU(MER_ERR_SUBMISSION, "cudaGraphLaunch", cudaGraphLaunch(hit->exec, s));
        CU(MER_ERR_READBACK_MAP, "cudaStreamSynchronize", cudaStreamSynchronize(s));
        b->ctr.kernel_launches += (uint64_t)hit->launches;
        b->ctr.selected_routed_experts += P;
        b->ctr.gpu_dispatch_attempts += P;
        b->ctr.hidden_upload_bytes += n_tokens * D * 4;
        b->ctr.readback_bytes += n_tokens * D * 4;
        int rc = check_device_status(b, b->h_u32[b->max_pairs], layer, expert);
        if (rc && rc != MER_ERR_NUMERICAL) {
          b->ctr.gpu_dispatch_failures += P;
          return rc;
        }
        b->ctr.gpu_dispatch_successes += P;
        return rc;
      }
    }
  }
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(x)", cudaMemcpyAsync(b->d_x, x, n_tokens * D * 4, cudaMemcpyHostToDevice, b->compute));
  int launches = 0;
  MoeDispatch d;
  int rc = enqueue_layer(b, layer, b->d_x, n_tokens, b->d_out, true, b->compute, &launches, &d);
  if (rc) return rc;
  const RouterDev &r = b->routers[layer].dev;
  size_t P = n_tokens * d.slots;
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(out)", cudaMemcpyAsync(out, b->d_out, n_tokens * D * 4, cudaMemcpyDeviceToHost, b->compute));
  if (ids) CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(ids)", cudaMemcpyAsync(b->h_u32, b->d_pair_expert, P * 4, cudaMemcpyDeviceToHost, b->compute));
  if (weights) CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(w)", cudaMemcpyAsync(b->h_f32, b->d_pair_weight, P * 4, cudaMemcpyDeviceToHost, b->compute));
  b->ctr.selected_routed_experts += P;
  rc = finish_host_call(b, layer, expert, launches, P);
  for (size_t t = 0; t < n_tokens; t++)
    for (uint32_t s = 0; s < r.top_k; s++) {
      if (ids) {
        uint32_t g = b->h_u32[t * d.slots + s];
        ids[t * r.top_k + s] = g == MER_NONE ? MER_NONE : g - r.id_base;
      }
      if (weights) weights[t * r.top_k + s] = b->h_f32[t * d.slots + s];
    }
  b->ctr.hidden_upload_bytes += n_tokens * D * 4;
  b->ctr.readback_bytes += n_tokens * D * 4 + (ids ? P * 4 : 0) + (weights ? P * 4 : 0);
  return rc;
}

namespace {
int layer_forward_device_locked(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, float *d_out, uint32_t *d_ids,
                                float *d_weights, cudaStream_t s);
}

MER_EXPORT int mer_moe_layer_forward_device(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, float *d_out,
                                            uint32_t *d_ids, float *d_weights, void *stream) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  if (!d_x || !d_out) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  return layer_forward_device_locked(b, layer, d_x, n_tokens, d_out, d_ids, d_weights, static_cast<cudaStream_t>(stream));
}

namespace {
int layer_forward_device_locked(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, float *d_out, uint32_t *d_ids,
                                float *d_weights, cudaStream_t s) {
  const uint32_t expert = MER_NONE;
  int launches = 0;
  size_t P = 0;
  const bool use_graph = b->graphs_ok && !b->timing_on && !(b->cfg.flags & MER_FLAG_NO_GRAPHS);
  bool replayed = false;
  if (use_graph) {
    auto it = b->routers.find(layer);
    if (it == b->routers.end()) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "no router installed for layer %u", layer);
    P = n_tokens * (it->second.dev.top_k + (it->second.dev.shared_expert_id != MER_NONE ? 1u : 0u));
    CU(MER_ERR_SUBMISSION, "wait for uploads", order_after_copies(b, s));  // outside any capture
    mer_backend::GraphEntry *hit = nullptr;
    for (auto &g : b->graphs)
      if (g.layer == layer && g.n_tokens == n_tokens && g.x == d_x && g.out == d_out && g.ids == d_ids && g.w == d_weights &&
          g.stream == s)
        hit = &g;
    if (!hit) {
      // first call with these arguments: capture the launch sequence once
      if (b->graphs.size() >= 256) drop_graphs(b);
      cudaGraph_t graph = nullptr;
      cudaGraphExec_t exec = nullptr;
      bool ok = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
      int rc = MER_OK;
      if (ok) {
        MoeDispatch d;
        rc = enqueue_layer(b, layer, d_x, n_tokens, d_out, true, s, &launches, &d, true);
        if (rc == MER_OK && d_ids) ok = cudaMemcpyAsync(d_ids, b->d_pair_expert, P * 4, cudaMemcpyDeviceToDevice, s) == cudaSuccess;
        if (rc == MER_OK && ok && d_weights)
          ok = cudaMemcpyAsync(d_weights, b->d_pair_weight, P * 4, cudaMemcpyDeviceToDevice, s) == cudaSuccess;
        cudaError_t ce = cudaStreamEndCapture(s, &graph);
        ok = ok && ce == cudaSuccess && graph != nullptr;
      }
      if (rc != MER_OK) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return rc;
      }
      if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
      if (graph) cudaGraphDestroy(graph);
      if (ok) {
        b->graphs.push_back({layer, n_tokens, d_x, d_out, d_ids, d_weights, s, exec, launches});
        hit = &b->graphs.back();
      } else {
        cudaGetLastError();
        b->graphs_ok = false;  // capture is not available here: plain launches from now on
      }
    }
    if (hit) {
      CU(MER_ERR_SUBMISSION, "cudaGraphLaunch", cudaGraphLaunch(hit->exec, s));
      launches = hit->launches;
      replayed = true;
    }
  }
  if (!replayed) {
    launches = 0;
    MoeDispatch d;
    int rc = enqueue_layer(b, layer, d_x, n_tokens, d_out, true, s, &launches, &d);
    if (rc) return rc;
    P = n_tokens * d.slots;
    // routing is exported as stored: [n_tokens x slots] global ids (slots = top_k + shared)
    if (d_ids) CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(ids)", cudaMemcpyAsync(d_ids, b->d_pair_expert, P * 4, cudaMemcpyDeviceToDevice, s));
    if (d_weights) CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(w)", cudaMemcpyAsync(d_weights, b->d_pair_weight, P * 4, cudaMemcpyDeviceToDevice, s));
  }
  CU(MER_ERR_SUBMISSION, "cudaEventRecord(stream use)", note_stream_use(b, s));
  b->ctr.kernel_launches += (uint64_t)launches;
  b->ctr.selected_routed_experts += P;
  b->ctr.gpu_dispatch_attempts += P;
  b->ctr.gpu_dispatch_successes += P;
  return MER_OK;
}
}  // namespace

// ---- pipelined host entry: upload, layer and read-back of consecutive calls overlap (one slot per call in flight)
namespace {
int ep_layer_forward_device_locked(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, float *d_out, cudaStream_t s);

int submit_impl(mer_backend *b, uint32_t layer, const float *x, size_t n_tokens, float *out, uint32_t slot, bool ep) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  if (!x || !out || slot >= MER_ASYNC_SLOTS) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer or slot >= %d", MER_ASYNC_SLOTS);
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  if (n_tokens == 0 || n_tokens > b->cfg.max_tokens)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "n_tokens %zu outside 1..=%u", n_tokens, b->cfg.max_tokens);
  auto it = b->routers.find(layer);
  if (it == b->routers.end()) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "no router installed for layer %u", layer);
  mer_backend::AsyncSlot &a = b->aslots[slot];
  if (a.in_flight) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "slot %u is still in flight: wait for it first", slot);
  cudaPointerAttributes ax{}, ao{};
  const bool pinned = cudaPointerGetAttributes(&ax, x) == cudaSuccess && ax.type == cudaMemoryTypeHost &&
                      cudaPointerGetAttributes(&ao, out) == cudaSuccess && ao.type == cudaMemoryTypeHost;
  cudaGetLastError();
  if (!pinned) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "the pipelined entry point needs pinned host buffers");
  const size_t D = b->cfg.d_model, bytes = n_tokens * D * 4;
  if (!a.d_x) {
    const size_t cap = (size_t)b->cfg.max_tokens * D * 4;
    CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(slot x)", cudaMalloc((void **)&a.d_x, cap));
    CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(slot out)", cudaMalloc((void **)&a.d_out, cap));
    CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(slot status)", cudaMalloc((void **)&a.d_status, 4));
    CU(MER_ERR_PHYSICAL_CAPACITY, "cudaHostAlloc(slot status)", cudaHostAlloc((void **)&a.h_status, 4, cudaHostAllocDefault));
    CU(MER_ERR_SUBMISSION, "cudaEventCreate", cudaEventCreateWithFlags(&a.ev_in, cudaEventDisableTiming));
    CU(MER_ERR_SUBMISSION, "cudaEventCreate", cudaEventCreateWithFlags(&a.ev_compute, cudaEventDisableTiming));
    CU(MER_ERR_SUBMISSION, "cudaEventCreate", cudaEventCreateWithFlags(&a.ev_out, cudaEventDisableTiming));
    if (!b->d2h) CU(MER_ERR_SUBMISSION, "cudaStreamCreate", cudaStreamCreateWithFlags(&b->d2h, cudaStreamNonBlocking));
  }
  // upload on the copy stream (the slot's previous layer call, waited for by the caller, is long done)
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(x)", cudaMemcpyAsync(a.d_x, x, bytes, cudaMemcpyHostToDevice, b->copy));
  CU(MER_ERR_SUBMISSION, "cudaEventRecord", cudaEventRecord(a.ev_in, b->copy));
  // the layer on the compute stream, then a copy of the status word it leaves (the next call resets the shared one)
  CU(MER_ERR_SUBMISSION, "cudaStreamWaitEvent", cudaStreamWaitEvent(b->compute, a.ev_in, 0));
  int rc = ep ? ep_layer_forward_device_locked(b, layer, a.d_x, n_tokens, a.d_out, b->compute)
              : layer_forward_device_locked(b, layer, a.d_x, n_tokens, a.d_out, nullptr, nullptr, b->compute);
  if (rc) return rc;
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(status)", cudaMemcpyAsync(a.d_status, b->d_status, 4, cudaMemcpyDeviceToDevice, b->compute));
  CU(MER_ERR_SUBMISSION, "cudaEventRecord", cudaEventRecord(a.ev_compute, b->compute));
  // read-back on its own stream
  CU(MER_ERR_SUBMISSION, "cudaStreamWaitEvent", cudaStreamWaitEvent(b->d2h, a.ev_compute, 0));
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(out)", cudaMemcpyAsync(out, a.d_out, bytes, cudaMemcpyDeviceToHost, b->d2h));
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(status)", cudaMemcpyAsync(a.h_status, a.d_status, 4, cudaMemcpyDeviceToHost, b->d2h));
  CU(MER_ERR_SUBMISSION, "cudaEventRecord", cudaEventRecord(a.ev_out, b->d2h));
  a.in_flight = true;
  a.layer = layer;
  a.pairs = n_tokens * (it->second.dev.top_k + (it->second.dev.shared_expert_id != MER_NONE ? 1u : 0u));
  b->ctr.hidden_upload_bytes += bytes;
  b->ctr.readback_bytes += bytes;
  return MER_OK;
}
}  // namespace

MER_EXPORT int mer_moe_layer_forward_submit(mer_backend *b, uint32_t layer, const float *x, size_t n_tokens, float *out, uint32_t slot) {
  return submit_impl(b, layer, x, n_tokens, out, slot, false);
}

MER_EXPORT int mer_ep_layer_forward_submit(mer_backend *b, uint32_t layer, const float *x, size_t n_tokens, float *out, uint32_t slot) {
  return submit_impl(b, layer, x, n_tokens, out, slot, true);
}

MER_EXPORT int mer_moe_layer_forward_wait(mer_backend *b, uint32_t slot) {
  if (!b || slot >= MER_ASYNC_SLOTS) return MER_ERR_INVALID_ARGUMENT;
  cudaEvent_t ev;
  uint32_t layer;
  {
    std::lock_guard<std::mutex> lock(b->mu);
    mer_backend::AsyncSlot &a = b->aslots[slot];
    if (!a.in_flight) return fail(b, MER_ERR_INVALID_ARGUMENT, 0, MER_NONE, "slot %u has nothing in flight", slot);
    ev = a.ev_out, layer = a.layer;
  }
  const uint32_t expert = MER_NONE;
  cudaError_t e = cudaEventSynchronize(ev);  // outside the lock: other threads may submit meanwhile
  std::lock_guard<std::mutex> lock(b->mu);
  mer_backend::AsyncSlot &a = b->aslots[slot];
  a.in_flight = false;
  if (e != cudaSuccess) return cuda_fail(b, MER_ERR_READBACK_MAP, layer, expert, "cudaEventSynchronize", e);
  int rc = check_device_status(b, *a.h_status, layer, expert);
  if (rc && rc != MER_ERR_NUMERICAL) {
    // the call was counted as a success when it was enqueued: move it
    if (b->ctr.gpu_dispatch_successes >= a.pairs) b->ctr.gpu_dispatch_successes -= a.pairs;
    b->ctr.gpu_dispatch_failures += a.pairs;
  }
  return rc;
}

// ------------------------------------------------------------------------ expert parallel

namespace {
size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

// Routed experts of the layer that live on this rank.
uint32_t ep_local_expert_count(const mer_backend *b, const RouterDev &r) {
  if (b->ep_owner_host.empty()) return b->ep.experts_per_rank;
  uint32_t n = 0;
  for (uint32_t e = r.id_base; e < r.id_base + r.num_experts && e < b->ep_owner_host.size(); e++) n += b->ep_owner_host[e] == b->ep.rank;
  return n;
}

// Dispatch over the tokens of all ranks whose routing (filtered to the local experts) is already in the workspace.
int ep_run_local_experts(mer_backend *b, uint32_t layer, const RouterDev &r, MoeDispatch &d, cudaStream_t s, int *launches, bool counted = false,
                         cudaEvent_t *ev = nullptr) {
  const uint32_t expert = MER_NONE;
  const uint32_t shared = r.shared_expert_id != MER_NONE ? 1u : 0u;
  d.slots = r.top_k + shared;
  d.n_groups = r.num_experts + shared;
  d.max_group_tokens = d.n_tokens;
  d.active_groups_hint = std::min(std::max(1u, ep_local_expert_count(b, r) + shared), d.n_tokens * d.slots);
  // of all ranks' pairs, about one in `world` lands on a local expert (the shared expert takes the rank's own tokens)
  d.expected_pairs = std::max<uint32_t>(1u, d.n_tokens * d.slots / b->ep.world);
  bind_ffn(b, d);
  CU(MER_ERR_SUBMISSION, "group kernel", launch_groups_layer(r, d, s, launches, counted));
  if (ev) cudaEventRecord(ev[1], s);
  CU(MER_ERR_SUBMISSION, "expert FFN kernels", run_ffn(b, d, s, launches, ev ? ev[2] : nullptr));
  return MER_OK;
}
}  // namespace

MER_EXPORT int mer_ep_init(mer_backend *b, const mer_ep_cfg *cfg) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = MER_NONE;
  if (!cfg) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null cfg");
  if (cfg->world == 0 || cfg->world > MER_EP_MAX_WORLD || cfg->rank >= cfg->world || cfg->experts_per_layer == 0 ||
      cfg->max_tokens_per_rank == 0)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "rank %u of %u, %u experts per layer, %u tokens per rank", cfg->rank,
                cfg->world, cfg->experts_per_layer, cfg->max_tokens_per_rank);
  if ((uint64_t)cfg->max_tokens_per_rank * cfg->world > b->cfg.max_tokens)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert,
                "the backend's max_tokens (%u) must cover the tokens of all ranks (%u x %u)", b->cfg.max_tokens,
                cfg->max_tokens_per_rank, cfg->world);
  std::lock_guard<std::mutex> lock(b->mu);
  if (b->ep_on) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "expert parallelism is already initialised");
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  const size_t D = b->cfg.d_model, S = b->cfg.max_top_k, Bm = cfg->max_tokens_per_rank, T = Bm * cfg->world;
  EpDev &ep = b->ep;
  ep = EpDev{};
  ep.rank = cfg->rank, ep.world = cfg->world;
  ep.experts_per_rank = (cfg->experts_per_layer + cfg->world - 1) / cfg->world;
  ep.wait_ns = (uint64_t)(cfg->wait_ms ? cfg->wait_ms : 2000u) * 1000000ull;
  ep.off_flags = 0;
  ep.off_x = 256;
  ep.off_ids = ep.off_x + round256(Bm * D * 4);
  b->ep_off_w = ep.off_ids + round256(Bm * S * 4);
  ep.off_y = b->ep_off_w + round256(Bm * S * 4);
  b->ep_bytes = ep.off_y + round256(T * S * D * 4);
  CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(exchange buffer)", cudaMalloc((void **)&b->ep_buf, b->ep_bytes));
  CU(MER_ERR_SUBMISSION, "cudaMemset(exchange buffer)", cudaMemset(b->ep_buf, 0, 256));
  ep.peer[ep.rank] = b->ep_buf;
  b->ep_cfg = *cfg;
  b->ep_on = true;
  b->ep_attached = cfg->world == 1;
  return MER_OK;
}

MER_EXPORT size_t mer_ep_exchange_bytes(mer_backend *b) { return b && b->ep_on ? b->ep_bytes : 0; }

MER_EXPORT int mer_ep_set_placement(mer_backend *b, const uint16_t *owner, size_t n_ids) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = MER_NONE;
  std::lock_guard<std::mutex> lock(b->mu);
  if (!b->ep_on) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "mer_ep_init has not been called");
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  // layers in flight and captured layer graphs hold the old rule
  CU(MER_ERR_SUBMISSION, "cudaDeviceSynchronize", cudaDeviceSynchronize());
  drop_graphs(b);
  if (!owner || n_ids == 0) {  // back to the contiguous rule
    b->ep_owner_host.clear();
    b->ep.owner = nullptr;
    return MER_OK;
  }
  if (n_ids > b->cfg.max_experts)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "%zu ids, the backend's id space has %u", n_ids, b->cfg.max_experts);
  for (size_t i = 0; i < n_ids; i++)
    if (owner[i] >= b->ep.world) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, (uint32_t)i, "owner %u of expert %zu outside the group of %u", owner[i], i, b->ep.world);
  if (!b->d_ep_owner) CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(placement table)", cudaMalloc((void **)&b->d_ep_owner, (size_t)b->cfg.max_experts * 2));
  // ids beyond the table keep the contiguous rule's answer, so that every id the kernels may look up has an entry
  std::vector<uint16_t> full(b->cfg.max_experts);
  const uint32_t E = b->ep_cfg.experts_per_layer, epr = b->ep.experts_per_rank;
  for (uint32_t i = 0; i < b->cfg.max_experts; i++) full[i] = i < n_ids ? owner[i] : (uint16_t)std::min((i % E) / epr, b->ep.world - 1);
  CU(MER_ERR_UPLOAD, "cudaMemcpy(placement table)", cudaMemcpy(b->d_ep_owner, full.data(), full.size() * 2, cudaMemcpyHostToDevice));
  b->ep_owner_host = std::move(full);
  b->ep.owner = b->d_ep_owner;
  return MER_OK;
}

MER_EXPORT int mer_ep_export_handle(mer_backend *b, void *handle_out) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = MER_NONE;
  if (!handle_out) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null handle buffer");
  std::lock_guard<std::mutex> lock(b->mu);
  if (!b->ep_on) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "mer_ep_init has not been called");
  static_assert(sizeof(cudaIpcMemHandle_t) == MER_EP_HANDLE_BYTES, "handle size");
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  cudaIpcMemHandle_t h;
  CU(MER_ERR_SUBMISSION, "cudaIpcGetMemHandle", cudaIpcGetMemHandle(&h, b->ep_buf));
  memcpy(handle_out, &h, sizeof h);
  return MER_OK;
}

MER_EXPORT int mer_ep_attach_handles(mer_backend *b, const void *handles, size_t n_handles) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = MER_NONE;
  std::lock_guard<std::mutex> lock(b->mu);
  if (!b->ep_on || !handles || n_handles != b->ep.world)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "expected the %u handles of an initialised group", b->ep_on ? b->ep.world : 0);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  for (uint32_t j = 0; j < b->ep.world; j++) {
    if (j == b->ep.rank || b->ep_opened[j]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const uint8_t *)handles + (size_t)j * MER_EP_HANDLE_BYTES, sizeof h);
    void *p = nullptr;
    CU(MER_ERR_SUBMISSION, "cudaIpcOpenMemHandle", cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    b->ep_opened[j] = p;
    b->ep.peer[j] = (uint8_t *)p;
  }
  b->ep_attached = true;
  return MER_OK;
}

MER_EXPORT int mer_ep_attach_pointers(mer_backend *b, void *const *exchange_buffers, size_t n) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = MER_NONE;
  std::lock_guard<std::mutex> lock(b->mu);
  if (!b->ep_on || !exchange_buffers || n != b->ep.world)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "expected the %u buffers of an initialised group", b->ep_on ? b->ep.world : 0);
  for (uint32_t j = 0; j < b->ep.world; j++) {
    if (j == b->ep.rank) continue;
    if (!exchange_buffers[j]) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null exchange buffer for rank %u", j);
    b->ep.peer[j] = (uint8_t *)exchange_buffers[j];
  }
  b->ep_attached = true;
  return MER_OK;
}

MER_EXPORT void *mer_ep_exchange_buffer(mer_backend *b) { return b && b->ep_on ? b->ep_buf : nullptr; }

MER_EXPORT int mer_router_route_device(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, uint32_t *d_ids,
                                       float *d_weights, void *stream) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  if (!d_x || !d_ids || !d_weights) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int launches = 0;
  MoeDispatch d;
  int rc = enqueue_layer(b, layer, d_x, n_tokens, b->d_out, false, s, &launches, &d);
  if (rc) return rc;
  const size_t P = n_tokens * d.slots;
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(ids)", cudaMemcpyAsync(d_ids, b->d_pair_expert, P * 4, cudaMemcpyDeviceToDevice, s));
  CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(w)", cudaMemcpyAsync(d_weights, b->d_pair_weight, P * 4, cudaMemcpyDeviceToDevice, s));
  CU(MER_ERR_SUBMISSION, "cudaEventRecord(stream use)", note_stream_use(b, s));
  b->ctr.kernel_launches += (uint64_t)launches;
  return MER_OK;
}

MER_EXPORT int mer_ep_local_experts_forward_device(mer_backend *b, uint32_t layer, const float *d_x_all, const uint32_t *d_ids_all,
                                                   const float *d_weights_all, size_t n_tokens_all, size_t tokens_per_rank,
                                                   float *d_out_partial, void *stream) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  if (!d_x_all || !d_ids_all || !d_weights_all || !d_out_partial) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  std::lock_guard<std::mutex> lock(b->mu);
  if (!b->ep_on) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "mer_ep_init has not been called");
  auto it = b->routers.find(layer);
  if (it == b->routers.end()) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "no router installed for layer %u", layer);
  const RouterDev &r = it->second.dev;
  if (n_tokens_all == 0 || n_tokens_all > b->cfg.max_tokens || tokens_per_rank == 0 || n_tokens_all != tokens_per_rank * b->ep.world)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "%zu tokens in all, %zu per rank, %u ranks, at most %u", n_tokens_all,
                tokens_per_rank, b->ep.world, b->cfg.max_tokens);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int launches = 0;
  EpDev ep = b->ep;
  ep.top_k = r.top_k, ep.id_base = r.id_base, ep.tokens_per_rank = (uint32_t)tokens_per_rank;
  MoeDispatch d = base_dispatch(b);
  d.n_tokens = (uint32_t)n_tokens_all;
  d.x = d_x_all;
  d.out = d_out_partial;
  const uint32_t slots = r.top_k + (r.shared_expert_id != MER_NONE ? 1u : 0u);
  CU(MER_ERR_SUBMISSION, "cudaMemsetAsync(status)", cudaMemsetAsync(b->d_status, 0, 4, s));
  CU(MER_ERR_SUBMISSION, "wait for uploads", order_after_copies(b, s));
  CU(MER_ERR_SUBMISSION, "filter kernel",
     launch_ep_filter(ep, d_ids_all, d_weights_all, d.n_tokens * slots, slots, d.pair_expert, d.pair_weight, s, &launches));
  int rc = ep_run_local_experts(b, layer, r, d, s, &launches);
  if (rc) return rc;
  CU(MER_ERR_SUBMISSION, "combine kernel", launch_combine(d, s, &launches));
  CU(MER_ERR_SUBMISSION, "cudaEventRecord(stream use)", note_stream_use(b, s));
  b->ctr.kernel_launches += (uint64_t)launches;
  return MER_OK;
}

MER_EXPORT int mer_ep_layer_forward_device(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, float *d_out,
                                           void *stream) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  if (!d_x || !d_out) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  std::lock_guard<std::mutex> lock(b->mu);
  return ep_layer_forward_device_locked(b, layer, d_x, n_tokens, d_out, static_cast<cudaStream_t>(stream));
}

namespace {
// Enqueues the launch sequence of one expert-parallel layer (peer-memory exchange) on stream s.
int ep_enqueue(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, float *d_out, cudaStream_t s, int *launches_out,
               bool capturing) {
  const uint32_t expert = MER_NONE;
  if (!b->ep_on || !b->ep_attached)
    return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "the expert-parallel group is not initialised and attached");
  auto it = b->routers.find(layer);
  if (it == b->routers.end()) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "no router installed for layer %u", layer);
  const RouterDev &r = it->second.dev;
  if (n_tokens == 0 || n_tokens > b->ep_cfg.max_tokens_per_rank)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "n_tokens %zu outside 1..=%u per rank", n_tokens, b->ep_cfg.max_tokens_per_rank);
  if ((b->cfg.d_model & 3) != 0) return fail(b, MER_ERR_INELIGIBLE, layer, expert, "d_model must be a multiple of 4");
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  int launches = 0;
  const size_t D = b->cfg.d_model;
  const uint32_t shared = r.shared_expert_id != MER_NONE ? 1u : 0u, slots = r.top_k + shared;
  EpDev ep = b->ep;
  ep.top_k = r.top_k, ep.id_base = r.id_base, ep.tokens_per_rank = (uint32_t)n_tokens;
  float *x_pub = reinterpret_cast<float *>(b->ep_buf + ep.off_x);
  uint32_t *ids_pub = reinterpret_cast<uint32_t *>(b->ep_buf + ep.off_ids);
  float *w_own = reinterpret_cast<float *>(b->ep_buf + b->ep_off_w);
  // the epoch the flags carry lives in device memory and advances by one per signal: the same launch sequence can be replayed
  uint32_t *epoch_counter = reinterpret_cast<uint32_t *>(b->ep_buf + 128);
  // stage timers (plain launches only): router_gate = router + publish + signal + gather (with its wait for the peers) +
  // grouping; gate/up and down as on one GPU; combine = signal + wait for the peers + pull
  cudaEvent_t *ev = capturing ? nullptr : next_timing_set(b);
  if (ev) cudaEventRecord(ev[0], s);

  CU(MER_ERR_SUBMISSION, "cudaMemsetAsync(status)", cudaMemsetAsync(b->d_status, 0, 4, s));
  if (!capturing) CU(MER_ERR_SUBMISSION, "wait for uploads", order_after_copies(b, s));
  // publish this rank's tokens (RMSNorm'ed when the layer has a norm installed) and their routing
  const RouterEntry &re = it->second;
  RouterDev rl = r;
  const bool gated = re.d_shared_gate && r.shared_expert_id != MER_NONE;
  if (re.d_rms_w || gated)
    CU(MER_ERR_SUBMISSION, "pre-MoE kernel",
       launch_pre_moe(d_x, (uint32_t)n_tokens, (uint32_t)D, re.d_rms_w, re.rms_eps, gated ? re.d_shared_gate : nullptr, x_pub, b->d_shared_scale, s,
                      &launches));
  if (!re.d_rms_w) CU(MER_ERR_SUBMISSION, "cudaMemcpyAsync(x)", cudaMemcpyAsync(x_pub, d_x, n_tokens * D * 4, cudaMemcpyDeviceToDevice, s));
  if (gated) rl.shared_scale = b->d_shared_scale;
  MoeDispatch dr = base_dispatch(b);
  dr.n_tokens = (uint32_t)n_tokens;
  dr.slots = slots;
  dr.n_groups = r.num_experts + shared;
  dr.x = x_pub;
  dr.pair_expert = ids_pub;
  dr.pair_weight = w_own;
  CU(MER_ERR_SUBMISSION, "router kernel", launch_router(rl, dr, b->cfg.max_tokens, s, &launches, false));
  // pull the tokens that hit a local expert, run the local experts over them
  MoeDispatch d = base_dispatch(b);
  d.n_tokens = (uint32_t)(n_tokens * ep.world);
  d.x = b->d_x;
  d.out = d_out;
  // per-pair outputs go to the home rank of their token: the GEMM kernels' down epilogue stores them there, the other
  // kernel families fill the local array (d.y) and a copy kernel moves the rows
  for (uint32_t j = 0; j < ep.world; j++) d.push_y[j] = ep.peer[j] + ep.off_y;
  d.push_tokens_per_rank = (uint32_t)n_tokens;
  d.slots = slots;
  const bool counted = groups_layer_on_grid(d);  // a large dispatch: the gather kernel does the grouping's count step
  CU(MER_ERR_SUBMISSION, "gather kernel",
     launch_ep_gather(ep, epoch_counter, (uint32_t)D, slots, b->d_x, d.pair_expert, d.pair_weight, b->d_status,
                      counted ? d.group_count : nullptr, r.num_experts, s, &launches));
  d.fuse_reduce = 1;  // the peers read final per-pair outputs, and only those of the local experts exist
  int rc = ep_run_local_experts(b, layer, r, d, s, &launches, counted, ev);
  if (rc) return rc;
  CU(MER_ERR_SUBMISSION, "partial-sum kernel", launch_reduce_parts(d, s, &launches));
  if (!d.gemm_bn) CU(MER_ERR_SUBMISSION, "push kernel", launch_ep_push_rows(d, s, &launches));
  if (ev) cudaEventRecord(ev[3], s);
  // weighted sum in slot order, every pair's output read from the rank that owns its expert
  CU(MER_ERR_SUBMISSION, "combine kernel",
     launch_ep_combine(ep, epoch_counter, (uint32_t)D, slots, ids_pub, w_own, (re.layer_flags & MER_LAYER_RESIDUAL) ? d_x : nullptr, d_out, b->d_status, s,
                       &launches));
  if (ev) cudaEventRecord(ev[4], s);
  *launches_out = launches;
  return MER_OK;
}

int ep_layer_forward_device_locked(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, float *d_out, cudaStream_t s) {
  const uint32_t expert = MER_NONE;
  int launches = 0;
  const void *ep_tag = reinterpret_cast<const void *>(uintptr_t(2));  // marks expert-parallel graphs in the cache
  bool replayed = false;
  if (b->graphs_ok && !b->timing_on && !(b->cfg.flags & MER_FLAG_NO_GRAPHS) && b->ep_on && b->ep_attached) {
    CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
    CU(MER_ERR_SUBMISSION, "wait for uploads", order_after_copies(b, s));  // outside any capture
    mer_backend::GraphEntry *hit = nullptr;
    for (auto &g : b->graphs)
      if (g.layer == layer && g.n_tokens == n_tokens && g.x == d_x && g.out == d_out && g.ids == ep_tag && g.stream == s) hit = &g;
    if (!hit) {
      if (b->graphs.size() >= 256) drop_graphs(b);
      cudaGraph_t graph = nullptr;
      cudaGraphExec_t exec = nullptr;
      int rc = MER_OK;
      bool ok = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
      if (ok) {
        rc = ep_enqueue(b, layer, d_x, n_tokens, d_out, s, &launches, true);
        cudaError_t ce = cudaStreamEndCapture(s, &graph);
        ok = ce == cudaSuccess && graph != nullptr;
      }
      if (rc != MER_OK) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return rc;
      }
      if (ok) ok = cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess;
      if (graph) cudaGraphDestroy(graph);
      if (ok) {
        b->graphs.push_back({layer, n_tokens, d_x, d_out, ep_tag, nullptr, s, exec, launches});
        hit = &b->graphs.back();
      } else {
        cudaGetLastError();
        b->graphs_ok = false;  // capture is not available here: plain launches from now on
      }
    }
    if (hit) {
      CU(MER_ERR_SUBMISSION, "cudaGraphLaunch", cudaGraphLaunch(hit->exec, s));
      launches = hit->launches;
      replayed = true;
    }
  }
  if (!replayed) {
    int rc = ep_enqueue(b, layer, d_x, n_tokens, d_out, s, &launches, false);
    if (rc) return rc;
  }
  CU(MER_ERR_SUBMISSION, "cudaEventRecord(stream use)", note_stream_use(b, s));
  b->ctr.kernel_launches += (uint64_t)launches;
  auto it = b->routers.find(layer);
  if (it != b->routers.end())
    b->ctr.selected_routed_experts += n_tokens * (it->second.dev.top_k + (it->second.dev.shared_expert_id != MER_NONE ? 1u : 0u));
  return MER_OK;
}}  // namespace

MER_EXPORT int mer_stream_check(mer_backend *b, uint32_t layer, void *stream) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t expert = MER_NONE;
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(status)",
     cudaMemcpyAsync(b->h_u32 + b->max_pairs, b->d_status, 4, cudaMemcpyDeviceToHost, s));
  CU(MER_ERR_READBACK_MAP, "cudaStreamSynchronize", cudaStreamSynchronize(s));
  return check_device_status(b, b->h_u32[b->max_pairs], layer, expert);
}

MER_EXPORT int mer_dequant_projection_f32(mer_backend *b, uint32_t expert_id, int projection, float *out) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = expert_id;
  if (!out || projection < 0 || projection > 2) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "bad projection or null out");
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  int rc = require_resident(b, layer, expert_id);
  if (rc) return rc;
  size_t n = (size_t)b->cfg.d_model * b->cfg.d_ff;
  if (!b->d_dequant) CU(MER_ERR_PHYSICAL_CAPACITY, "cudaMalloc(dequant)", cudaMalloc((void **)&b->d_dequant, n * 4));
  CU(MER_ERR_SUBMISSION, "wait for uploads", order_after_copies(b, b->compute));
  if (b->packed) {
    CU(MER_ERR_SUBMISSION, "dequant kernel",
       launch_dequant_packed(b->cfg.dtype, b->h_expert_ptr[expert_id], projection, (uint32_t)b->cfg.d_model, (uint32_t)b->cfg.d_ff,
                             b->d_dequant, b->compute));
  } else {
    const uint8_t *src = b->h_expert_ptr[expert_id] + (size_t)projection * (b->expert_bytes / 3);
    CU(MER_ERR_SUBMISSION, "dequant kernel", launch_dequant(b->cfg.dtype, src, b->d_dequant, n, b->compute));
  }
  CU(MER_ERR_READBACK_MAP, "cudaMemcpyAsync(out)", cudaMemcpyAsync(out, b->d_dequant, n * 4, cudaMemcpyDeviceToHost, b->compute));
  CU(MER_ERR_READBACK_MAP, "cudaStreamSynchronize", cudaStreamSynchronize(b->compute));
  b->ctr.kernel_launches++;
  return MER_OK;
}

MER_EXPORT int mer_qualification_matvec(mer_backend *b, int32_t dtype, const void *weights, size_t weights_len, const float *input,
                                        size_t rows, size_t columns, size_t w_block_off, float *out) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  const uint32_t layer = 0, expert = MER_NONE;
  if (!weights || !input || !out) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "null pointer");
  if (dtype != MER_DTYPE_Q4_0 && dtype != MER_DTYPE_Q8_0) return fail(b, MER_ERR_INVALID_ARGUMENT, layer, expert, "unknown dtype");
  // validate_raw_case (q4_parity.rs:621-660)
  if (rows == 0 || columns == 0 || columns % MER_BLOCK_ELEMS != 0)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "invalid raw geometry rows=%zu columns=%zu", rows, columns);
  size_t bb = block_bytes(dtype), need = (w_block_off + rows * (columns / MER_BLOCK_ELEMS)) * bb;
  if (weights_len < need || weights_len % bb != 0)
    return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "raw weights have %zu bytes, require at least %zu complete blocks' worth",
                weights_len, need);
  for (size_t i = 0; i < columns; i++)
    if (!std::isfinite(input[i])) return fail(b, MER_ERR_VALIDATION_DISPATCH, layer, expert, "raw input contains a nonfinite value");
  std::lock_guard<std::mutex> lock(b->mu);
  CU(MER_ERR_SUBMISSION, "cudaSetDevice", cudaSetDevice(b->cfg.device));
  uint8_t *d_w = nullptr;
  float *d_in = nullptr, *d_o = nullptr;
  cudaError_t e = cudaMalloc((void **)&d_w, weights_len);
  if (e == cudaSuccess) e = cudaMalloc((void **)&d_in, columns * 4);
  if (e == cudaSuccess) e = cudaMalloc((void **)&d_o, rows * 4);
  if (e == cudaSuccess) e = cudaMemcpyAsync(d_w, weights, weights_len, cudaMemcpyHostToDevice, b->compute);
  if (e == cudaSuccess) e = cudaMemcpyAsync(d_in, input, columns * 4, cudaMemcpyHostToDevice, b->compute);
  if (e == cudaSuccess) e = launch_raw_matvec(dtype, d_w + w_block_off * bb, d_in, d_o, rows, columns, b->compute);
  if (e == cudaSuccess) e = cudaMemcpyAsync(out, d_o, rows * 4, cudaMemcpyDeviceToHost, b->compute);
  if (e == cudaSuccess) e = cudaStreamSynchronize(b->compute);
  cudaFree(d_w), cudaFree(d_in), cudaFree(d_o);
  if (e != cudaSuccess) return cuda_fail(b, MER_ERR_SUBMISSION, layer, expert, "raw qualification matvec", e);
  return MER_OK;
}

MER_EXPORT int mer_stage_timing_enable(mer_backend *b, int on) {
  if (!b) return MER_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(b->mu);
  cudaSetDevice(b->cfg.device);
  drain_timing(b);
  b->timing_on = on != 0;
  if (on) b->timing_acc = mer_stage_timings{};
  return MER_OK;
}

MER_EXPORT int mer_stage_timings_read(mer_backend *b, mer_stage_timings *out) {
  if (!b || !out) return MER_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(b->mu);
  cudaSetDevice(b->cfg.device);
  drain_timing(b);
  *out = b->timing_acc;
  return MER_OK;
}

MER_EXPORT int mer_last_error(mer_backend *b, mer_error_info *out) {
  if (!b || !out) return MER_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(b->mu);
  *out = b->err;
  return MER_OK;
}

MER_EXPORT int mer_snapshot(mer_backend *b, mer_counters *out) {
  if (!b || !out) return MER_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(b->mu);
  b->ctr.resident_experts = b->id2slot.size();
  b->ctr.resident_bytes = b->id2slot.size() * b->expert_bytes;
  *out = b->ctr;
  return MER_OK;
}

MER_EXPORT int mer_set_kernel_path(mer_backend *b, int path) {
  if (!b || path < 0 || path > 3) return MER_ERR_INVALID_ARGUMENT;
  std::lock_guard<std::mutex> lock(b->mu);
  if (path == 2 && !b->d_stream_scratch)
    return fail(b, MER_ERR_INELIGIBLE, 0, MER_NONE, "streaming kernels need d_model and d_ff to be multiples of 256");
  if (path == 3 && !b->d_gemm_scratch)
    return fail(b, MER_ERR_INELIGIBLE, 0, MER_NONE,
                "the GEMM kernels need d_model and d_ff to be multiples of 256 and a backend of at least %u tokens", 12u);
  b->kernel_path = path;
  drop_graphs(b);
  return MER_OK;
}

#include "mer_abi_ep_nccl.inc"
