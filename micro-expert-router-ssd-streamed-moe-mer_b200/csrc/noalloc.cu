// mer_expert_forward_noalloc: one expert's SwiGLU FFN for a few tokens without a backend handle and
// without allocating anything, for hosts that must not let a library allocate device memory on
// their behalf: an engine that has handed the whole device to its own pool and keeps an exact byte
// ledger of it, or a caller sitting in a latency-critical section where cudaMalloc's implicit
// device synchronisation is not acceptable.
//
// The intermediate silu(gate)*up vector and the small dispatch tables live in ONE file-scope device
// array that every GPU loading this library holds until exit (size below).  The array's name is only
// a host-side stand-in in host code, so its device address is fetched once per device with
// cudaGetSymbolAddress() while that device is current, and that pointer is what kernels receive.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/mer_b200.h"
#include "kernels.h"

#define MER_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t H_BYTES = (size_t)MER_NOALLOC_MAX_TOKENS * MER_NOALLOC_MAX_DIM * sizeof(float);  // silu(gate)*up rows
constexpr size_t TABLE_BYTES = 1024;  // expert pointer, group table, offsets, perm, ids, weights, status
constexpr size_t SCRATCH_BYTES = H_BYTES + TABLE_BYTES;

static __device__ __align__(256) unsigned char g_noalloc_scratch[SCRATCH_BYTES];

// Layout of the table area (offsets from the start of the scratch array).
constexpr size_t OFF_EXPERT_PTR = H_BYTES;         // const uint8_t* [1]
constexpr size_t OFF_GROUP = H_BYTES + 64;         // uint32 [1]
constexpr size_t OFF_OFFSETS = H_BYTES + 128;      // uint32 [2]
constexpr size_t OFF_PERM = H_BYTES + 192;         // uint32 [MAX_TOKENS]
constexpr size_t OFF_PAIR_EXPERT = H_BYTES + 320;  // uint32 [MAX_TOKENS]
constexpr size_t OFF_PAIR_WEIGHT = H_BYTES + 448;  // float  [MAX_TOKENS]
constexpr size_t OFF_STATUS = H_BYTES + 576;       // uint32 [1]

// Device code may name the array directly.  Everything a call depends on is rewritten here, because
// the array still holds whatever the previous call left in it.
__global__ void k_noalloc_setup(const uint8_t *expert, uint32_t n_tokens) {
  unsigned char *s = g_noalloc_scratch;
  if (threadIdx.x == 0) {
    *reinterpret_cast<const uint8_t **>(s + OFF_EXPERT_PTR) = expert;
    *reinterpret_cast<uint32_t *>(s + OFF_GROUP) = 0;  // the one group runs "expert id" 0 of a 1-entry table
    reinterpret_cast<uint32_t *>(s + OFF_OFFSETS)[0] = 0;
    reinterpret_cast<uint32_t *>(s + OFF_OFFSETS)[1] = n_tokens;
    *reinterpret_cast<uint32_t *>(s + OFF_STATUS) = 0;
  }
  if (threadIdx.x < MER_NOALLOC_MAX_TOKENS) {
    reinterpret_cast<uint32_t *>(s + OFF_PERM)[threadIdx.x] = threadIdx.x;
    reinterpret_cast<uint32_t *>(s + OFF_PAIR_EXPERT)[threadIdx.x] = threadIdx.x < n_tokens ? 0u : MER_NONE;
    reinterpret_cast<float *>(s + OFF_PAIR_WEIGHT)[threadIdx.x] = 1.0f;
  }
}

constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
unsigned char *g_scratch_ptr[MAX_DEVICES] = {};

void set_err(char *err, size_t err_len, const char *msg) {
  if (err && err_len) snprintf(err, err_len, "%s", msg);
}

}  // namespace

MER_EXPORT int mer_expert_forward_noalloc(int32_t dtype, uint64_t d_model, uint64_t d_ff, const void *d_expert_blob,
                                          const float *d_x, size_t n_tokens, float *d_out, float swiglu_limit, void *stream,
                                          char *err, size_t err_len) {
  if (dtype != MER_DTYPE_Q4_0 && dtype != MER_DTYPE_Q8_0) {
    set_err(err, err_len, "unknown dtype");
    return MER_ERR_INVALID_ARGUMENT;
  }
  if (!d_expert_blob || !d_x || !d_out) {
    set_err(err, err_len, "null pointer");
    return MER_ERR_INVALID_ARGUMENT;
  }
  if (n_tokens == 0 || n_tokens > MER_NOALLOC_MAX_TOKENS || d_model == 0 || d_ff == 0 || d_model > MER_NOALLOC_MAX_DIM ||
      d_ff > MER_NOALLOC_MAX_DIM) {
    if (err && err_len)
      snprintf(err, err_len,
               "size beyond the fixed scratch of the no-allocation entry point: n_tokens=%zu (max %d), d_model=%llu, d_ff=%llu "
               "(max %d each)",
               n_tokens, MER_NOALLOC_MAX_TOKENS, (unsigned long long)d_model, (unsigned long long)d_ff, MER_NOALLOC_MAX_DIM);
    return MER_ERR_VALIDATION_DISPATCH;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    cudaGetLastError();
    set_err(err, err_len, "no current CUDA device");
    return MER_ERR_DEVICE_LOST;
  }
  unsigned char *scratch;
  {
    // First call on this device: resolve the device address of the static array (no allocation).
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_ptr[dev]) {
      unsigned char *p = nullptr;
      cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_noalloc_scratch);
      if (e != cudaSuccess || !p) {
        if (err && err_len) snprintf(err, err_len, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return MER_ERR_RUNTIME_INVARIANT;
      }
      g_scratch_ptr[dev] = p;
    }
    scratch = g_scratch_ptr[dev];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MoeDispatch d{};
  d.expert_ptr = reinterpret_cast<const uint8_t *const *>(scratch + OFF_EXPERT_PTR);
  d.max_experts = 1;
  d.dtype = dtype;
  d.D = (uint32_t)d_model;
  d.F = (uint32_t)d_ff;
  d.n_tokens = (uint32_t)n_tokens;
  d.slots = 1;
  d.n_groups = 1;
  d.x = d_x;
  d.pair_expert = reinterpret_cast<uint32_t *>(scratch + OFF_PAIR_EXPERT);
  d.pair_weight = reinterpret_cast<float *>(scratch + OFF_PAIR_WEIGHT);
  d.group_expert = reinterpret_cast<uint32_t *>(scratch + OFF_GROUP);
  d.offsets = reinterpret_cast<uint32_t *>(scratch + OFF_OFFSETS);
  d.perm = reinterpret_cast<uint32_t *>(scratch + OFF_PERM);
  d.h = reinterpret_cast<float *>(scratch);  // the scratch proper
  d.y = d_out;                               // one slot per token: the per-pair output is the result
  d.out = d_out;
  d.status = reinterpret_cast<uint32_t *>(scratch + OFF_STATUS);
  d.swiglu_limit = swiglu_limit;
  d.packed = 0;  // the caller's blob is the reference's flat gate||up||down stream
  k_noalloc_setup<<<1, 32, 0, s>>>(static_cast<const uint8_t *>(d_expert_blob), (uint32_t)n_tokens);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = launch_ffn_generic(d, s, nullptr, nullptr);
  if (e != cudaSuccess) {
    if (err && err_len) snprintf(err, err_len, "kernel launch failed: %s", cudaGetErrorString(e));
    return MER_ERR_SUBMISSION;
  }
  return MER_OK;
}
