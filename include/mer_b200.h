/*
 * mer_b200.h -- C ABI of the B200 (sm_100a) routed quantized SwiGLU expert-FFN backend.
 *
 * This is the boundary a Micro-Expert-Router host binds (Rust `extern "C"`, ctypes, cgo ...):
 * plain pointers and sizes, status codes, no exceptions, no framework types.  Every entry
 * point cites the reference interface it stands in for (paths relative to
 * rust-engine/src/ of the reference).
 *
 * Conventions
 *  - Every function returns a mer_status (0 = ok) unless stated otherwise; on failure
 *    mer_last_error() describes the typed error {layer, expert_id, kind, detail}, the
 *    C form of GpuExpertDispatchError (backend/mod.rs:423-428).
 *  - The caller owns every buffer it passes, for the duration of the call only.
 *  - "host" entry points take host pointers, copy through pinned staging buffers and
 *    return after the result is in the caller's buffer (the reference's boundary is
 *    synchronous: backend/mod.rs:2726-2790).  "_device" entry points take device
 *    pointers and enqueue on a caller-supplied stream without synchronising.
 *  - A backend may be used from several host threads; calls on one backend serialise.
 *  - There is no CPU fallback anywhere behind this ABI (RoutedExpertGpuFailurePolicy::
 *    StrictFailClosed, engine.rs:996-1000): a call either runs on the GPU or fails.
 *  - Expert weights are never passed per call.  They are admitted once
 *    (mer_expert_admit) into an HBM slot keyed by (expert_id, generation), exactly the
 *    residency contract of GpuBackend::routed_expert_matmul (backend/mod.rs:3856-4018).
 *  - Expert ids are global: layer * experts_per_layer + local (model.rs:2717-2725).
 */
#ifndef MER_B200_H
#define MER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MER_ABI_VERSION 1

/* WeightDtype subset on this path (inference.rs:725-747, kernels/mod.rs:74-75). */
#define MER_DTYPE_Q4_0 0 /* 18-byte blocks: f16 d + 16 nibble bytes, value = d * (q - 8) */
#define MER_DTYPE_Q8_0 1 /* 34-byte blocks: f16 d + 32 int8,         value = d * q       */

/* Status / error kinds.  1..9 are GpuExpertDispatchErrorKind (backend/mod.rs:349-361) in
 * declaration order; the rest extend it for a C boundary. */
typedef enum mer_status {
  MER_OK = 0,
  MER_ERR_RESIDENCY_MISS = 1,
  MER_ERR_PHYSICAL_CAPACITY = 2,
  MER_ERR_UPLOAD = 3,
  MER_ERR_VALIDATION_DISPATCH = 4,
  MER_ERR_SUBMISSION = 5,
  MER_ERR_READBACK_CHANNEL = 6,
  MER_ERR_READBACK_MAP = 7,
  MER_ERR_DEVICE_LOST = 8,
  MER_ERR_RUNTIME_INVARIANT = 9,
  MER_ERR_INELIGIBLE = 10,       /* GpuExpertBatchDispatchOutcome::Ineligible (backend/mod.rs:454-458) */
  MER_ERR_TIMEOUT = 11,          /* a bounded device-side wait gave up */
  MER_ERR_INVALID_ARGUMENT = 12, /* NULL pointer, zero size, unknown layer ... */
  MER_ERR_NUMERICAL = 13         /* non-finite routing scores latched by the device status word */
} mer_status;

/* Device status word bits (same meaning as the reference's gpu_native status bits,
 * backend/gpu_native.rs:25-41): latched by kernels instead of trapping. */
#define MER_DEVSTAT_RESIDENCY_MISS 0x1u   /* a routed expert had no current HBM slot */
#define MER_DEVSTAT_NONFINITE_ROUTER 0x2u /* softmax row was non-finite and fell back to uniform */
#define MER_DEVSTAT_TIMEOUT 0x4u          /* bounded wait expired */
#define MER_DEVSTAT_SHORT_SELECTION 0x8u  /* fewer than top_k finite scores */

#define MER_EXPERT_NONE 0xFFFFFFFFu /* id written for an unfilled top-k slot / "no shared expert" */

/* Scoring function of the router (ScoringFunc, gating.rs:94-97). */
#define MER_SCORE_SOFTMAX 0
#define MER_SCORE_SIGMOID 1

/* mer_backend_cfg.flags */
#define MER_FLAG_NO_GRAPHS 0x1u /* mer_moe_layer_forward_device: always launch kernel by kernel (no CUDA graph replay) */

/* mer_expert_admit flags. */
#define MER_ADMIT_ANCHOR 0x1u /* Anchor Core entry: never evicted (expert_cache.rs:798-828) */
#define MER_ADMIT_ASYNC 0x2u  /* return once the side-stream copy is enqueued */
#define MER_ADMIT_NO_READER_WAIT 0x4u /* the copy stream does not wait for the layers in flight: the caller guarantees that none of
                                         them reads the slot this admission (or the eviction it causes) rewrites.  That is the case
                                         when every expert those layers may route to was looked up (mer_gpu_cache_get /
                                         mer_expert_touch) after the eviction's victims: the admission's H2D copy then overlaps their
                                         kernels instead of queueing behind them */

typedef struct mer_backend mer_backend;

/* ModelShape + EngineOptions subset (engine.rs:958-965, 1008-1109) + [gpu_cache] sizing. */
typedef struct mer_backend_cfg {
  int32_t device;               /* CUDA ordinal */
  int32_t dtype;                /* MER_DTYPE_* */
  uint64_t d_model;
  uint64_t d_ff;
  uint64_t vram_capacity_bytes; /* byte budget of the HBM expert slot arena */
  uint32_t max_experts;         /* size of the global expert id space */
  uint32_t max_tokens;          /* largest token batch of one layer call */
  uint32_t max_top_k;           /* largest top_k (+1 if a shared expert is used) */
  float swiglu_limit;           /* GPT-OSS gate clamp; <= 0 or non-finite = off (inference.rs:86-112) */
  uint32_t flags;               /* MER_FLAG_* */
  uint32_t reserved;
} mer_backend_cfg;

/* LinearGate (gating.rs:118-143). */
typedef struct mer_router_cfg {
  uint32_t num_experts;
  uint32_t top_k;
  int32_t scoring_func;         /* MER_SCORE_* */
  int32_t normalise_topk;
  uint32_t n_group;             /* 0/1 = no grouping */
  uint32_t topk_group;
  float routed_scaling_factor;
  uint32_t shared_expert_id;    /* global id of an always-on expert added with weight 1, or MER_EXPERT_NONE
                                   (SharedExpert, transformer.rs:2094-2238) */
  const float *correction_bias; /* host [num_experts] or NULL; selection only (gating.rs:406-416) */
  const float *logit_bias;      /* host [num_experts] or NULL; harness extension: added to the logits */
} mer_router_cfg;

/* GpuExpertDispatchError (backend/mod.rs:423-428). */
typedef struct mer_error_info {
  uint32_t layer;
  uint32_t expert_id;
  int32_t kind; /* mer_status */
  uint32_t device_status;
  char detail[256];
} mer_error_info;

/* RoutedExpertExecutionSnapshot (engine.rs:943-951) + GpuExpertIoSnapshot /
 * GpuExpertMemorySnapshot ledgers (backend/mod.rs:466-547). */
typedef struct mer_counters {
  uint64_t selected_routed_experts;
  uint64_t gpu_dispatch_attempts;
  uint64_t gpu_dispatch_successes;
  uint64_t gpu_dispatch_failures;
  uint64_t batch_calls;
  uint64_t kernel_launches;
  uint64_t expert_uploads;
  uint64_t expert_upload_bytes;
  uint64_t hidden_upload_bytes;
  uint64_t readback_bytes;
  uint64_t evictions;
  uint64_t resident_experts;
  uint64_t resident_bytes;
  uint64_t arena_bytes;
  uint64_t slot_stride_bytes;
  uint64_t slot_count;
} mer_counters;

int mer_abi_version(void);
const char *mer_error_kind_name(int kind); /* GpuExpertDispatchErrorKind Display, backend/mod.rs:403-418 */
/* expert_weight_bytes_for (inference.rs:1096-1114): bytes of one gate||up||down blob. */
uint64_t mer_expert_bytes(int32_t dtype, uint64_t d_model, uint64_t d_ff);
/* routed_expert_gpu_compatibility (backend/mod.rs:4691-4720), extended to Q8_0. 0 = eligible. */
int mer_routed_expert_compatibility(int32_t dtype, uint64_t d_model, uint64_t d_ff);

/* resolve_execution_context factory seam (backend/mod.rs:5514-5594): builds the backend
 * one BackendBox arm would own. */
int mer_backend_create(const mer_backend_cfg *cfg, mer_backend **out);
void mer_backend_destroy(mer_backend *b);
int mer_backend_synchronize(mer_backend *b);

/* ---- residency: the VRAM tier (expert_cache.rs:734-1350 logical tier + physical registry
 * backend/mod.rs:3856-4018; slot layout after backend/gpu_native.rs:68-75, 1607). ---- */

/* demand_admit_lru + build_expert_entry_q4_0 (expert_cache.rs:1281-1340, backend/mod.rs:2612):
 * copies the header-stripped blob (ExpertResident::data, expert_cache.rs:202) from host memory
 * through pinned staging on the copy stream into an HBM slot.  Evicts least-recently-used
 * non-anchor slots when the arena is full.  A generation older than the resident one is a
 * stale requester (MER_ERR_RESIDENCY_MISS); the same generation is a no-op. */
int mer_expert_admit(mer_backend *b, uint32_t expert_id, uint64_t generation, const void *host_blob,
                     size_t bytes, uint32_t flags);
/* Same, from a blob already in device memory (device-to-device copy or repack on the copy stream, which is not
 * ordered after the caller's streams: the blob must be complete when the call is made, and must stay untouched
 * until the admission has finished: mer_backend_synchronize, or a synchronous admit). */
int mer_expert_admit_device(mer_backend *b, uint32_t expert_id, uint64_t generation,
                            const void *device_blob, size_t bytes, uint32_t flags);
/* retire_key_if_present (backend/mod.rs:3893): frees the slot if (id, generation) is current. */
int mer_expert_retire(mer_backend *b, uint32_t expert_id, uint64_t generation);
/* contains_generation (expert_cache.rs:909): 1 if (id, generation) is resident, else 0. */
int mer_expert_contains_generation(mer_backend *b, uint32_t expert_id, uint64_t generation);

/* ---- logical VRAM tier: GpuExpertCache (expert_cache.rs:734-1350), the host-side policy that decides which
 * experts are admitted to the GPU.  Pure bookkeeping: no CUDA call, usable without a device.  Two byte-budgeted
 * regions are cut from `capacity_bytes` by `anchor_ratio` (clamped to [0, 1]; expert_cache.rs:798-828): the Anchor
 * Core, whose entries are never evicted, and the LRU Edge, which admits foreground demand and evicts least recently
 * used.  Generations start at 1, grow monotonically, are allocated before any eviction and are never reused; the
 * physical slots of mer_expert_admit are keyed by (expert_id, generation), so a stale physical copy is detected
 * with mer_gpu_cache_contains_generation exactly as backend/mod.rs:3884-3912 does.  The payload itself stays with
 * the caller; `payload_tag` is an opaque 64-bit identity stored with the admission (the reference keeps an
 * Arc<GpuResident>).  Calls that may evict report the evicted ids (up to max_evicted; *n_evicted is the true count)
 * so that the caller retires their physical slots. ---- */
typedef struct mer_gpu_cache mer_gpu_cache;

#define MER_REGION_NONE 0
#define MER_REGION_ANCHOR 1
#define MER_REGION_LRU 2
/* GpuLookup (expert_cache.rs:629-646) */
#define MER_LOOKUP_MISS 0
#define MER_LOOKUP_ANCHOR_HIT 1
#define MER_LOOKUP_LRU_HIT 2
/* GpuHotPromotionOutcome (expert_cache.rs:667-702); the first three change state and count as promotions */
#define MER_HOT_MOVED_LRU_TO_ANCHOR 0
#define MER_HOT_INSTALLED_ANCHOR 1
#define MER_HOT_INSTALLED_LRU 2
#define MER_HOT_ALREADY_ANCHOR 3
#define MER_HOT_ALREADY_LRU_ANCHOR_FULL 4
#define MER_HOT_PAYLOAD_REQUIRED 5
#define MER_HOT_NO_CAPACITY 6
#define MER_HOT_GENERATION_EXHAUSTED 7
/* GpuDemandAdmissionPreflight / demand_admit_lru results and GpuDemandAdmissionError (expert_cache.rs:649-665) */
#define MER_DEMAND_ALREADY_ADMITTED 0 /* preflight: AlreadyAdmitted; demand_admit_lru: Ok(false) */
#define MER_DEMAND_NEEDS_PAYLOAD 1    /* preflight only */
#define MER_DEMAND_ADMITTED 2         /* demand_admit_lru: Ok(true) */
#define MER_DEMAND_ERR_EMPTY_PAYLOAD (-1)
#define MER_DEMAND_ERR_EXCEEDS_LRU_CAPACITY (-2)
#define MER_DEMAND_ERR_GENERATION_EXHAUSTED (-3)

/* GpuAdmission (expert_cache.rs:600-623) */
typedef struct mer_gpu_admission {
  uint32_t expert_id;
  uint32_t region; /* MER_REGION_* */
  uint64_t generation;
  uint64_t bytes;
  uint64_t payload_tag;
} mer_gpu_admission;

typedef struct mer_gpu_cache_stats {
  uint64_t anchor_capacity_bytes, lru_capacity_bytes;
  uint64_t anchor_used_bytes, lru_used_bytes, used_bytes; /* used_bytes = logical admitted bytes (expert_cache.rs:835) */
  uint64_t anchor_len, lru_len;
  uint64_t promotions, hits, misses; /* mer_promotions_total, mer_gpu_cache_hits_total, mer_gpu_cache_misses_total */
  uint64_t next_generation;
  uint64_t promote_after_hits;
  uint64_t pending_promotions, rearmed_promotions;
} mer_gpu_cache_stats;

/* GpuExpertCache::new (expert_cache.rs:798-828) */
int mer_gpu_cache_create(uint64_t capacity_bytes, float anchor_ratio, uint64_t promote_after_hits, mer_gpu_cache **out);
void mer_gpu_cache_destroy(mer_gpu_cache *c);
/* get (expert_cache.rs:864-879): the only call that counts a hit or a miss and refreshes LRU recency. Returns MER_LOOKUP_*. */
int mer_gpu_cache_get(mer_gpu_cache *c, uint32_t expert_id, mer_gpu_admission *out);
/* current_admission / contains / contains_generation (expert_cache.rs:884-912): no counters, no recency. Return 1 / 0. */
int mer_gpu_cache_current_admission(mer_gpu_cache *c, uint32_t expert_id, mer_gpu_admission *out);
int mer_gpu_cache_contains(mer_gpu_cache *c, uint32_t expert_id);
int mer_gpu_cache_contains_generation(mer_gpu_cache *c, uint32_t expert_id, uint64_t generation);
/* should_promote / claim_promotion / cancel_promotion (expert_cache.rs:918-952): one claim per threshold edge
 * (ram_hits == promote_after_hits) and one more after every logical eviction of the id; never two pending. */
int mer_gpu_cache_should_promote(mer_gpu_cache *c, uint64_t ram_hits);
int mer_gpu_cache_claim_promotion(mer_gpu_cache *c, uint32_t expert_id, uint64_t ram_hits);
void mer_gpu_cache_cancel_promotion(mer_gpu_cache *c, uint32_t expert_id);
/* promote_hot_existing / promote_hot_sync (expert_cache.rs:962-1046). Return MER_HOT_*. */
int mer_gpu_cache_promote_hot_existing(mer_gpu_cache *c, uint32_t expert_id);
int mer_gpu_cache_promote_hot_sync(mer_gpu_cache *c, uint32_t expert_id, uint64_t bytes, uint64_t payload_tag, uint32_t *evicted,
                                   size_t max_evicted, size_t *n_evicted, uint64_t *generation);
/* promote_sync (expert_cache.rs:1116-1192): warm-up admission, Anchor first when it fits, else LRU with eviction. 1 / 0. */
int mer_gpu_cache_promote_sync(mer_gpu_cache *c, uint32_t expert_id, uint64_t bytes, uint64_t payload_tag, uint32_t *evicted,
                               size_t max_evicted, size_t *n_evicted, uint64_t *generation);
/* try_promote_lru_no_evict (expert_cache.rs:1208-1249): speculative, never evicts, never uses the Anchor Core. 1 / 0. */
int mer_gpu_cache_try_promote_lru_no_evict(mer_gpu_cache *c, uint32_t expert_id, uint64_t bytes, uint64_t payload_tag,
                                           uint64_t *generation);
/* demand_admission_preflight (expert_cache.rs:1251-1270): side-effect free. Returns MER_DEMAND_*. */
int mer_gpu_cache_demand_admission_preflight(mer_gpu_cache *c, uint32_t expert_id, uint64_t payload_bytes);
/* demand_admit_lru (expert_cache.rs:1281-1340): foreground demand enters the LRU Edge; the generation is allocated
 * before victims are evicted; the Anchor Core is never touched; an existing admission changes nothing. MER_DEMAND_*. */
int mer_gpu_cache_demand_admit_lru(mer_gpu_cache *c, uint32_t expert_id, uint64_t bytes, uint64_t payload_tag, uint32_t *evicted,
                                   size_t max_evicted, size_t *n_evicted, uint64_t *generation);
/* Drops (expert_id, generation) from whichever region holds it (the host retired the expert). 1 if it was current. */
int mer_gpu_cache_remove(mer_gpu_cache *c, uint32_t expert_id, uint64_t generation);
int mer_gpu_cache_stats_read(mer_gpu_cache *c, mer_gpu_cache_stats *out);
/* Moves the generation counter forward (never back): lets a host resume a numbering, and tests reach exhaustion. */
int mer_gpu_cache_set_next_generation(mer_gpu_cache *c, uint64_t next_generation);
/* bit 0: a promotion request is pending for the id; bit 1: the id may claim one more after its eviction. */
int mer_gpu_cache_marker_state(mer_gpu_cache *c, uint32_t expert_id);

/* ---- the logical tier driving the physical one: Engine::ensure_gpu_admission / the GPU arm of moe_step_inner
 * (engine.rs:2382-2429, 5494-5643) followed by GpuBackend's lazy upload keyed by (id, generation)
 * (backend/mod.rs:3856-4018).  Both calls leave `cache` and the backend's slots consistent: ids the policy evicts are
 * retired from their slots before the new payload is uploaded.  Flags as mer_expert_admit (MER_ADMIT_ASYNC). ---- */
/* Foreground demand for `expert_id`: preflight, demand_admit_lru, retire the victims, upload under the new generation.
 * An id that is already admitted logically but has no physical copy of its current generation is uploaded again under
 * that generation.  *generation receives the current generation.  Oversized payload: MER_ERR_PHYSICAL_CAPACITY. */
int mer_expert_demand_admit(mer_backend *b, mer_gpu_cache *cache, uint32_t expert_id, const void *host_blob, size_t bytes,
                            uint32_t flags, uint64_t *generation);
/* Threshold-driven promotion (the background promotion task of engine.rs install_gpu_cache): moves an LRU admission
 * into the Anchor Core, or installs an absent expert (host_blob required then).  Returns MER_OK and the
 * MER_HOT_* outcome in *outcome; the slot of an anchored expert is never evicted. */
int mer_expert_hot_promote(mer_backend *b, mer_gpu_cache *cache, uint32_t expert_id, const void *host_blob, size_t bytes,
                           uint32_t flags, int *outcome);
/* Routing feedback for hosts whose router runs on the device: counts one mer_gpu_cache_get per id (hits, misses, LRU
 * recency; `cache` may be NULL) and refreshes the physical slots' recency. */
int mer_expert_touch(mer_backend *b, mer_gpu_cache *cache, const uint32_t *expert_ids, size_t n);

/* ---- on-disk formats around the expert path: the Unified Tensor Header in front of an expert blob
 * (tensor_header.rs:9-27: UTH1, 64 bytes; tensor_header.rs:256-283: UTH2, 128 bytes, one byte range per projection;
 * both followed by zero padding up to block_align when flag bit 0 is set) and the dataset's metadata.json
 * (main.rs:9096-9114).  Host-only parsing, no device needed. ---- */
#define MER_UTH_KIND_NONE 0 /* legacy blob: no header, the payload is the whole buffer */
#define MER_UTH_KIND_UTH1 1
#define MER_UTH_KIND_UTH2 2
typedef struct mer_uth_projection { /* ProjectionRange (tensor_header.rs:144-150); offsets relative to the payload */
  uint32_t uth_dtype_id;            /* UthDtypeId (tensor_header.rs:75-89): 4 = Q4_0, 5 = Q8_0, ... */
  uint32_t weights;
  uint64_t offset, len;
} mer_uth_projection;
typedef struct mer_uth_info {
  uint32_t kind;          /* MER_UTH_KIND_* */
  uint32_t version;
  uint32_t uth_dtype_id;  /* UTH1: the blob's dtype id; UTH2: 10 (mixed) */
  int32_t dtype;          /* MER_DTYPE_* when this library runs it (UTH2: all three projections alike), else -1 */
  uint32_t shape_rank, flags;
  uint32_t shape[4];      /* UTH1: [d_ff, d_model, 3, 0] for a SwiGLU expert (tensor_header.rs:456) */
  uint64_t d_model, d_ff;
  uint64_t payload_offset, payload_bytes; /* where the weights start inside the buffer, and what is left from there */
  mer_uth_projection proj[3];             /* UTH2: gate, up, down */
} mer_uth_info;
/* TensorHeader::strip / MixedExpertHeader::strip (tensor_header.rs:528-545, 376-391).  Best effort like the reference:
 * a buffer without a valid header is reported as MER_UTH_KIND_NONE, never as an error. */
int mer_uth_probe(const void *bytes, size_t len, size_t block_align, mer_uth_info *out);
/* The same for a blob of `len` bytes of which only the first `have` (at least 128) are in memory: a file's header region. */
int mer_uth_probe_prefix(const void *bytes, size_t have, uint64_t len, size_t block_align, mer_uth_info *out);
/* TensorHeader::for_swiglu_expert + write_padded (tensor_header.rs:419-470, 489-499): header + padding; *written = bytes
 * needed (MER_ERR_PHYSICAL_CAPACITY when cap is smaller). */
int mer_uth1_write(int32_t dtype, uint64_t d_model, uint64_t d_ff, size_t block_align, void *dst, size_t cap, size_t *written);
/* MixedExpertHeader::to_bytes + write_padded (tensor_header.rs:256-295). */
int mer_uth2_write(uint64_t d_model, uint64_t d_ff, const mer_uth_projection *proj /*[3]*/, size_t block_align, void *dst,
                   size_t cap, size_t *written);
typedef struct mer_dataset_info { /* the keys of metadata.json a loader needs; absent keys stay 0 / "" / -1 */
  uint64_t format_version, num_experts, d_model, d_ff, expert_size, maximum_payload_bytes, block_align, experts_written;
  uint64_t num_layers, experts_per_layer, top_k;
  int32_t dtype; /* MER_DTYPE_* or -1 */
  char dtype_name[16], q4_0_layout[32], conversion_mode[32];
} mer_dataset_info;
int mer_dataset_metadata_parse(const char *json, size_t len, mer_dataset_info *out);
/* The loader: expert_<id>.bin (gguf_loader.rs:782) -> HBM slot.  Reads the file in chunks straight into the pinned
 * staging buffers (no intermediate copy), strips a UTH1 / UTH2 header (UTH2: the three ranges are gathered into the
 * gate||up||down order), checks dtype and shape against the backend, and admits under (expert_id, generation) like
 * mer_expert_admit.  block_align = the dataset's (metadata.json; 4096 by default). */
int mer_expert_admit_file(mer_backend *b, uint32_t expert_id, uint64_t generation, const char *path, size_t block_align,
                          uint32_t flags);

/* ---- router: LinearGate::new / with_routing (gating.rs:149-238). ---- */
int mer_router_install(mer_backend *b, uint32_t layer, const float *host_weights /*[E x D]*/,
                       const mer_router_cfg *cfg);
/* ---- the steps either side of the MoE block, per layer (optional; install after the layer's router):
 *   rms_weight  pre-MoE RMSNorm (RmsNorm::forward_inplace, transformer.rs:52-95): router and experts read
 *               xn = x * (1 / sqrt(mean(x^2) + rms_eps)) * rms_weight instead of x (moe_pre, transformer.rs:2493-2518);
 *   shared_gate the shared expert's sigmoid gate vector (SharedExpert::gate_inp, transformer.rs:2101-2103, 2224-2237):
 *               its output is mixed in with weight sigmoid(shared_gate . xn) instead of 1;
 *   MER_LAYER_RESIDUAL  the combine writes out = (x + sum over routed slots) + shared expert, the order of
 *               moe_accumulated_into + add_residual_into (transformer.rs:2559-2574, model.rs:2742-2763); out may alias x.
 * The whole-layer entry points (mer_moe_layer_forward*, mer_ep_layer_forward*) honour them; entry points whose
 * routing comes from the caller do not.  Both vectors are host pointers of d_model floats, or NULL. ---- */
#define MER_LAYER_RESIDUAL 0x1u
typedef struct mer_layer_cfg {
  const float *rms_weight;
  const float *shared_gate;
  float rms_eps;
  uint32_t flags;
} mer_layer_cfg;
int mer_layer_install(mer_backend *b, uint32_t layer, const mer_layer_cfg *cfg);

/* LinearGate::route_with_scratch (gating.rs:395-476) for n_tokens rows of x (host).
 * ids/weights are [n_tokens x top_k]; unfilled slots get MER_EXPERT_NONE / 0. Ids are local. */
int mer_router_route(mer_backend *b, uint32_t layer, const float *x, size_t n_tokens,
                     uint32_t *ids, float *weights);

/* ---- compute, host buffers ---- */

/* BackendBox::routed_expert_matmul (backend/mod.rs:4421-4441): one token through one expert,
 * f16 in / f16 out (TensorView, backend/mod.rs:327-339). x and out are d_model binary16 values. */
int mer_routed_expert_matmul(mer_backend *b, uint32_t layer, uint32_t expert_id, const uint16_t *x,
                             size_t d_model, size_t d_ff, uint16_t *out);
/* BackendBox::routed_expert_matmul_batch_q4 (backend/mod.rs:4401-4418): one token through n
 * experts in one call, outputs [n x d_model] f16 in slot order, duplicates allowed.  The
 * reference accepts exactly 8 Q4_0 experts; here any n in 1..=max_top_k and both dtypes.
 * Returns MER_ERR_INELIGIBLE (nothing ran; the caller keeps its scalar path) when n is out of
 * range; a failure after dispatch started is never replayed (engine.rs:6624-6642). */
int mer_routed_expert_matmul_batch(mer_backend *b, uint32_t layer, const uint32_t *expert_ids,
                                   size_t n, const uint16_t *x, size_t d_model, size_t d_ff,
                                   uint16_t *out);
/* f32 form of the same dispatch (the parity target): n_tokens rows through one expert. */
int mer_routed_expert_forward_f32(mer_backend *b, uint32_t layer, uint32_t expert_id,
                                  const float *x, size_t n_tokens, float *out);
/* Engine::moe_step_weighted_into (engine.rs:5174-5643, compute block): routing given, one
 * token, out[d] = sum over slots in order of weights[s] * expert_s(x)[d], zero weights skipped. */
int mer_moe_step_weighted_into(mer_backend *b, uint32_t layer, const float *x,
                               const uint32_t *expert_ids, const float *weights, size_t n_slots,
                               float *out);
/* The whole path for n_tokens rows (host): router top-k -> permute -> gate/up + SiLU*mul ->
 * down -> weighted combine (+ shared expert).  moe_pre + moe_step + moe_combine,
 * transformer.rs:2493-2574, batched over tokens.  ids/weights (optional) receive the routing. */
int mer_moe_layer_forward(mer_backend *b, uint32_t layer, const float *x, size_t n_tokens,
                          float *out, uint32_t *ids, float *weights);

/* ---- compute, device buffers, asynchronous on `stream` (a cudaStream_t) ----
 * The launch sequence of a call is captured into a CUDA graph the first time a (layer, n_tokens,
 * pointers, stream) combination is seen and replayed afterwards (one cudaGraphLaunch per call), so
 * the first call with new arguments must not itself be inside a stream capture.  The backend's
 * workspace is shared: calls on different streams must not overlap. */
int mer_moe_layer_forward_device(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens,
                                 float *d_out, uint32_t *d_ids, float *d_weights, void *stream);

/* dequantize_q4_0_to_f32 / dequantize_q8_0_to_f32 (inference.rs:852-868, 963-979) on the
 * resident copy: projection 0 = gate, 1 = up, 2 = down; out is d_model*d_ff floats (host). */
int mer_dequant_projection_f32(mer_backend *b, uint32_t expert_id, int projection, float *out);

/* GpuBackend::qualification_q4_0_matvec (backend/mod.rs:3532-3700): raw block-stream matvec used
 * by the parity qualification cases (q4_parity.rs:470-572).  out[r] = sum_c W[r,c] * input[c] with
 * row r starting at block w_block_off + r * columns/32.  Owns ephemeral device buffers, touches
 * neither residency nor the dispatch counters.  All pointers are host pointers. */
int mer_qualification_matvec(mer_backend *b, int32_t dtype, const void *weights, size_t weights_len,
                             const float *input, size_t rows, size_t columns, size_t w_block_off,
                             float *out);

/* ---- no-allocation variant (no counterpart in the reference) ----
 * One expert's SwiGLU FFN for up to MER_NOALLOC_MAX_TOKENS rows, for callers that cannot let a
 * library allocate device memory: no backend handle, no cudaMalloc/cudaFree, no allocating library
 * call.  d_expert_blob is the flat gate||up||down block stream in device memory; d_x is
 * [n_tokens x d_model] f32 and d_out [n_tokens x d_model] f32, both device pointers; work is enqueued
 * on `stream` of the CURRENT device and not synchronised.  The silu(gate)*up intermediate lives in a
 * fixed array inside the library (about 0.5 MiB, held by every GPU that loads the library until the
 * process exits), so: sizes beyond the maxima below are refused with MER_ERR_VALIDATION_DISPATCH and a
 * message in `err`; all calls on one GPU share that array, so two calls that overlap on the GPU (two
 * streams, two threads) race - serialise them; the first call on a device looks the array's address
 * up, so make that first call outside any stream capture.  Runs the generic fp32 kernels. */
#define MER_NOALLOC_MAX_TOKENS 8
#define MER_NOALLOC_MAX_DIM 16384
int mer_expert_forward_noalloc(int32_t dtype, uint64_t d_model, uint64_t d_ff, const void *d_expert_blob,
                               const float *d_x, size_t n_tokens, float *d_out, float swiglu_limit,
                               void *stream, char *err, size_t err_len);

/* ---- pipelined host entry: mer_moe_layer_forward for callers that keep several independent token batches in
 * flight (a serving loop over micro-batches; the reference's engine overlaps SSD reads with compute the same way,
 * engine.rs:5174-5643, and has no device boundary to pipeline).  x and out must be pinned host memory and stay
 * untouched until the wait.  submit() enqueues upload (copy stream), layer (compute stream) and read-back (its own
 * stream) and returns; wait() blocks until out holds the result and returns the call's typed status.  A slot
 * (0 .. MER_ASYNC_SLOTS-1) carries one call at a time; calls on different slots overlap. ---- */
#define MER_ASYNC_SLOTS 4
int mer_moe_layer_forward_submit(mer_backend *b, uint32_t layer, const float *x, size_t n_tokens,
                                 float *out, uint32_t slot);
int mer_moe_layer_forward_wait(mer_backend *b, uint32_t slot);
/* The same for the expert-parallel layer of this rank's tokens (mer_ep_layer_forward_device in the middle); every
 * rank must submit the same sequence of calls.  Waited for with mer_moe_layer_forward_wait. */
int mer_ep_layer_forward_submit(mer_backend *b, uint32_t layer, const float *x, size_t n_tokens,
                                float *out, uint32_t slot);

/* ---- per-stage device timing: StageTimings (stage_timing.rs:6-29) with the reference's stage
 * names, measured with CUDA events on the stream each layer call is enqueued on. ---- */
typedef struct mer_stage_timings {
  uint64_t samples;                    /* layer calls accumulated */
  double router_gate_ms;               /* router logits + scoring + top-k + token->expert grouping */
  double expert_gate_up_kernel_ms;     /* gate/up dequant-matvec + SiLU*mul (whole expert FFN when one kernel does both) */
  double expert_down_kernel_ms;        /* down projection (0 when fused into the kernel above) */
  double moe_weighted_combination_ms;  /* weighted top-k combine */
  double expert_compute_ms;            /* gate/up + down */
} mer_stage_timings;
/* Turns event recording around each stage on (1) or off (0); turning it on clears the accumulators. */
int mer_stage_timing_enable(mer_backend *b, int on);
/* Waits for the recorded events and returns the accumulated per-stage times. */
int mer_stage_timings_read(mer_backend *b, mer_stage_timings *out);

/* ---- expert parallelism: one backend per GPU, the experts of every layer split contiguously over
 * the ranks (rank j owns the local indices [j*ceil(E/world), (j+1)*ceil(E/world))), a shared expert
 * replicated on every rank and run for the rank's own tokens.  Stands in for the reference's only
 * multi-node expert placement, ShardRouter / RouteExperts (distributed.rs, docs/distributed.md:16-50:
 * router node computes top-k, fans out per shard, sums weighted outputs; a shard that times out
 * contributes zero and is counted).  Here a peer that does not answer within wait_ms latches
 * MER_DEVSTAT_TIMEOUT and the call fails with MER_ERR_TIMEOUT at the next mer_stream_check.
 * The backend's max_tokens must cover world * max_tokens_per_rank; a rank admits only its own
 * experts (plus the shared expert). ---- */
#define MER_EP_MAX_WORLD 16
#define MER_EP_HANDLE_BYTES 64
typedef struct mer_ep_cfg {
  uint32_t rank, world;
  uint32_t experts_per_layer;   /* routed experts per layer (E) */
  uint32_t max_tokens_per_rank; /* every rank brings the same number of tokens to a step, at most this many */
  uint32_t wait_ms;             /* limit of every device-side wait on a peer; 0 = 2000 */
  uint32_t reserved;
} mer_ep_cfg;
/* Allocates this rank's exchange buffer (tokens, routing, per-pair expert outputs, arrival flags). */
int mer_ep_init(mer_backend *b, const mer_ep_cfg *cfg);
size_t mer_ep_exchange_bytes(mer_backend *b);
/* Expert placement.  By default rank j holds the local expert indices [j * ceil(E / N), (j + 1) * ceil(E / N)) of every
 * layer.  A table owner[global expert id] = rank (n_ids entries from id 0; the same table on every rank) replaces that
 * rule for every exchange mode, e.g. a placement balanced by measured expert popularity: the reference's ShardRouter
 * maps experts to nodes by id % num_nodes (distributed.rs), which is as blind to popularity as the contiguous split.
 * Which experts a rank admits is the host's side of the same table.  NULL / 0 restores the default.  Synchronises the
 * device; call between steps, on every rank before the next layer call. */
int mer_ep_set_placement(mer_backend *b, const uint16_t *owner, size_t n_ids);
/* One process per GPU: export the exchange buffer as a 64-byte CUDA IPC handle; after the host has
 * exchanged the handles of all ranks (rank order), attach maps the peers' buffers. */
int mer_ep_export_handle(mer_backend *b, void *handle_out);
int mer_ep_attach_handles(mer_backend *b, const void *handles, size_t n_handles);
/* One process driving several GPUs with peer access enabled: pass the buffers directly. */
void *mer_ep_exchange_buffer(mer_backend *b);
int mer_ep_attach_pointers(mer_backend *b, void *const *exchange_buffers, size_t n);
/* LinearGate::route for n_tokens device rows: ids [n x slots] global ids, weights [n x slots]
 * (slots = top_k + shared); asynchronous on `stream`. */
int mer_router_route_device(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens,
                            uint32_t *d_ids, float *d_weights, void *stream);
/* Collectives run by the host (all-gather of x / ids / weights in rank order, reduce-scatter of the
 * partial outputs): runs the experts of this rank over the tokens of all ranks and writes
 * d_out_partial [n_tokens_all x d_model] = sum over the local pairs of weight * expert(x). */
int mer_ep_local_experts_forward_device(mer_backend *b, uint32_t layer, const float *d_x_all,
                                        const uint32_t *d_ids_all, const float *d_weights_all,
                                        size_t n_tokens_all, size_t tokens_per_rank,
                                        float *d_out_partial, void *stream);
/* The whole layer for this rank's n_tokens rows with the exchange done by the kernels through peer
 * memory: route, publish, pull the tokens that hit a local expert, run the local experts -- the down
 * projection stores every pair's output straight into the exchange buffer of the token's home rank --
 * and sum each token's rows in slot order (same order as a single GPU).  Every rank must make the
 * same sequence of calls with the same n_tokens. */
int mer_ep_layer_forward_device(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens,
                                float *d_out, void *stream);
/* ---- the same layer with NCCL all-to-all dispatch and combine (the library calls NCCL itself; it binds libnccl.so.2
 * at run time, MER_ERR_INELIGIBLE when none can be loaded).  One rank obtains a 128-byte ncclUniqueId, the host hands
 * it to every rank (any transport), every rank calls mer_ep_nccl_init after mer_ep_init (collective).  Per layer:
 * route the rank's tokens, pack every (token, slot) pair into the send segment of the rank that owns its expert,
 * all-gather the row counts, grouped ncclSend / ncclRecv of only the rows that hit a peer's experts (+ their expert
 * ids), local experts over the received rows, the outputs back the same way, weighted sum in slot order.  The call
 * synchronises `stream` once (the exchange is sized on the host from the counts) and is otherwise asynchronous.
 * Stands in for RouteExperts(layer, expert_ids, hidden) -> ffn_out of the reference's shard protocol
 * (proto/route_experts.proto, distributed.rs).
 * Teardown: mer_backend_destroy of a backend that joined the exchange destroys its communicator, which waits for the
 * peers' (ncclCommDestroy): every rank must destroy its backend, and in the same order relative to any other NCCL
 * communicator the host tears down, or the two teardowns wait for each other. ---- */
#define MER_NCCL_ID_BYTES 128
int mer_ep_nccl_unique_id(void *id_out /*[MER_NCCL_ID_BYTES]*/);
int mer_ep_nccl_init(mer_backend *b, const void *unique_id);
int mer_ep_layer_forward_a2a_device(mer_backend *b, uint32_t layer, const float *d_x, size_t n_tokens, float *d_out, void *stream);
/* Synchronises `stream` and turns the device status word into a typed error (for _device calls). */
int mer_stream_check(mer_backend *b, uint32_t layer, void *stream);

/* ---- introspection ---- */
int mer_last_error(mer_backend *b, mer_error_info *out);
int mer_snapshot(mer_backend *b, mer_counters *out);
/* Selects the kernel family: 0 = automatic (streaming kernels for a few tokens per expert, the
 * tcgen05 GEMM kernels from a mean of 12 tokens per expert), 1 = generic fp32 kernels (any shape),
 * 2 = streaming tensor-core kernels, 3 = tcgen05 GEMM kernels (2 and 3: block-aligned shapes).
 * For qualification runs. */
int mer_set_kernel_path(mer_backend *b, int path);

#ifdef __cplusplus
}
#endif
#endif /* MER_B200_H */
