// On-disk formats around the expert path (host only, no CUDA call): the Unified Tensor Header that
// gguf-convert puts in front of an expert blob (UTH1, 64 bytes; UTH2, 128 bytes with one byte range per
// projection; both page-padded so that the payload starts on a block boundary) and the dataset's
// metadata.json.  Layouts follow tensor_header.rs:9-27, 256-283, 419-545 and main.rs:9096-9114 of the
// reference.  mer_expert_admit_file (mer_abi.cu) uses the probe to find the payload inside a file.
#include <cctype>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/mer_b200.h"

#define MER_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t UTH1_BYTES = 64, UTH2_BYTES = 128;
constexpr uint32_t UTH_FLAG_PAGE_ALIGNED_PAYLOAD = 1u;
constexpr uint8_t UTH_DTYPE_Q4_0 = 4, UTH_DTYPE_Q8_0 = 5, UTH_DTYPE_MIXED = 10, UTH_DTYPE_LAST = 10;

uint16_t le16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
uint32_t le32(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24); }
uint64_t le64(const uint8_t *p) { return (uint64_t)le32(p) | ((uint64_t)le32(p + 4) << 32); }
void put16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v, p[1] = (uint8_t)(v >> 8); }
void put32(uint8_t *p, uint32_t v) {
  for (int i = 0; i < 4; i++) p[i] = (uint8_t)(v >> (8 * i));
}
void put64(uint8_t *p, uint64_t v) {
  for (int i = 0; i < 8; i++) p[i] = (uint8_t)(v >> (8 * i));
}

int backend_dtype(uint8_t uth_id) { return uth_id == UTH_DTYPE_Q4_0 ? MER_DTYPE_Q4_0 : uth_id == UTH_DTYPE_Q8_0 ? MER_DTYPE_Q8_0 : -1; }
uint8_t uth_dtype(int dtype) { return dtype == MER_DTYPE_Q4_0 ? UTH_DTYPE_Q4_0 : UTH_DTYPE_Q8_0; }

size_t padded_prefix(size_t header, uint32_t flags, size_t block_align) {
  if ((flags & UTH_FLAG_PAGE_ALIGNED_PAYLOAD) && block_align > 0) return header + (block_align - header % block_align) % block_align;
  return header;
}

}  // namespace

// TensorHeader::strip / MixedExpertHeader::strip (tensor_header.rs:528-545, 376-391): a blob without a valid
// header is a legacy blob and is returned unchanged (kind 0, payload = the whole buffer).
MER_EXPORT int mer_uth_probe(const void *bytes_, size_t len, size_t block_align, mer_uth_info *out) {
  return mer_uth_probe_prefix(bytes_, len, len, block_align, out);
}

// The same for a blob of `len` bytes of which only the first `have` are in memory (the header region of a file).
MER_EXPORT int mer_uth_probe_prefix(const void *bytes_, size_t have, uint64_t len, size_t block_align, mer_uth_info *out) {
  if (!bytes_ || !out || have > len) return MER_ERR_INVALID_ARGUMENT;
  const uint8_t *b = static_cast<const uint8_t *>(bytes_);
  memset(out, 0, sizeof *out);
  out->dtype = -1;
  out->payload_bytes = len;
  if (have >= UTH1_BYTES && memcmp(b, "UTH1", 4) == 0) {
    const uint16_t version = le16(b + 4);
    const uint8_t dt = b[6], rank = b[7];
    if (version == 0 || version > 1 || dt > UTH_DTYPE_LAST || rank == 0 || rank > 4) return MER_OK;  // not a header we know: legacy
    const uint32_t flags = le32(b + 44);
    const size_t prefix = padded_prefix(UTH1_BYTES, flags, block_align);
    if (prefix > len) return MER_OK;
    out->kind = MER_UTH_KIND_UTH1;
    out->version = version;
    out->uth_dtype_id = dt;
    out->dtype = backend_dtype(dt);
    out->shape_rank = rank;
    for (int i = 0; i < 4; i++) out->shape[i] = le32(b + 8 + 4 * i);
    // for_swiglu_expert records [d_ff, d_model, 3] (tensor_header.rs:456)
    out->d_ff = out->shape[0];
    out->d_model = out->shape[1];
    out->flags = flags;
    out->payload_offset = prefix;
    out->payload_bytes = len - prefix;
    return MER_OK;
  }
  if (have >= UTH2_BYTES && memcmp(b, "UTH2", 4) == 0) {
    if (le16(b + 4) != 2 || le16(b + 6) != 3) return MER_OK;
    mer_uth_info h{};
    h.kind = MER_UTH_KIND_UTH2;
    h.version = 2;
    h.uth_dtype_id = UTH_DTYPE_MIXED;
    h.dtype = -1;
    h.d_model = le32(b + 8);
    h.d_ff = le32(b + 12);
    h.flags = le32(b + 16);
    for (int i = 0; i < 3; i++) {
      const uint8_t *p = b + 24 + 24 * i;
      if (p[1] != i || p[0] > UTH_DTYPE_LAST) return MER_OK;  // role byte must be gate, up, down in order
      h.proj[i].uth_dtype_id = p[0];
      h.proj[i].offset = le64(p + 4);
      h.proj[i].len = le64(p + 12);
      h.proj[i].weights = le32(p + 20);
    }
    const size_t prefix = padded_prefix(UTH2_BYTES, h.flags, block_align);
    if (prefix > len) return MER_OK;
    const uint64_t payload = len - prefix;
    // MixedExpertHeader::validate (tensor_header.rs:195-254): non-zero shape and ranges, inside the payload, disjoint
    if (h.d_model == 0 || h.d_ff == 0) return MER_OK;
    for (int i = 0; i < 3; i++) {
      const uint64_t off = h.proj[i].offset, n = h.proj[i].len;
      if (h.proj[i].uth_dtype_id == UTH_DTYPE_MIXED || n == 0 || off + n < off || off + n > payload) return MER_OK;
      for (int j = 0; j < i; j++) {
        const uint64_t o2 = h.proj[j].offset, n2 = h.proj[j].len;
        if (off < o2 + n2 && o2 < off + n) return MER_OK;
      }
    }
    if (h.proj[0].uth_dtype_id == h.proj[1].uth_dtype_id && h.proj[1].uth_dtype_id == h.proj[2].uth_dtype_id)
      h.dtype = backend_dtype(h.proj[0].uth_dtype_id);
    h.payload_offset = prefix;
    h.payload_bytes = payload;
    *out = h;
    return MER_OK;
  }
  return MER_OK;
}

// TensorHeader::for_swiglu_expert + write_padded (tensor_header.rs:419-470, 489-499).
MER_EXPORT int mer_uth1_write(int32_t dtype, uint64_t d_model, uint64_t d_ff, size_t block_align, void *dst_, size_t cap, size_t *written) {
  if (!dst_ || !written || (dtype != MER_DTYPE_Q4_0 && dtype != MER_DTYPE_Q8_0)) return MER_ERR_INVALID_ARGUMENT;
  const size_t total = padded_prefix(UTH1_BYTES, UTH_FLAG_PAGE_ALIGNED_PAYLOAD, block_align);
  *written = total;
  if (cap < total) return MER_ERR_PHYSICAL_CAPACITY;
  uint8_t *d = static_cast<uint8_t *>(dst_);
  memset(d, 0, total);
  memcpy(d, "UTH1", 4);
  put16(d + 4, 1);
  d[6] = uth_dtype(dtype);
  d[7] = 3;
  put32(d + 8, (uint32_t)d_ff), put32(d + 12, (uint32_t)d_model), put32(d + 16, 3);
  put32(d + 32, 16), put32(d + 36, 16), put32(d + 40, 64);  // advisory tile hints of the reference's writer
  put32(d + 44, UTH_FLAG_PAGE_ALIGNED_PAYLOAD);
  return MER_OK;
}

// MixedExpertHeader::to_bytes + write_padded (tensor_header.rs:256-295) for three ranges given relative to the payload.
MER_EXPORT int mer_uth2_write(uint64_t d_model, uint64_t d_ff, const mer_uth_projection *proj, size_t block_align, void *dst_, size_t cap,
                              size_t *written) {
  if (!dst_ || !written || !proj) return MER_ERR_INVALID_ARGUMENT;
  const size_t total = padded_prefix(UTH2_BYTES, UTH_FLAG_PAGE_ALIGNED_PAYLOAD, block_align);
  *written = total;
  if (cap < total) return MER_ERR_PHYSICAL_CAPACITY;
  uint8_t *d = static_cast<uint8_t *>(dst_);
  memset(d, 0, total);
  memcpy(d, "UTH2", 4);
  put16(d + 4, 2), put16(d + 6, 3);
  put32(d + 8, (uint32_t)d_model), put32(d + 12, (uint32_t)d_ff), put32(d + 16, UTH_FLAG_PAGE_ALIGNED_PAYLOAD);
  for (int i = 0; i < 3; i++) {
    uint8_t *p = d + 24 + 24 * i;
    p[0] = (uint8_t)proj[i].uth_dtype_id, p[1] = (uint8_t)i;
    put64(p + 4, proj[i].offset), put64(p + 12, proj[i].len), put32(p + 20, proj[i].weights);
  }
  return MER_OK;
}

// ---- metadata.json (main.rs:9096-9114; the converter writes the same keys): a flat JSON object.  Only the
// keys the loader needs are read; unknown keys, nested values included, are skipped.
namespace {
struct Json {
  const char *p, *end;
  void ws() {
    while (p < end && isspace((unsigned char)*p)) p++;
  }
  bool lit(char c) {
    ws();
    if (p < end && *p == c) return p++, true;
    return false;
  }
  bool string(std::string *out) {
    ws();
    if (p >= end || *p != '"') return false;
    p++;
    std::string s;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        p++;
        s.push_back(*p == 'n' ? '\n' : *p == 't' ? '\t' : *p);  // \uXXXX does not occur in the keys and values read here
      } else {
        s.push_back(*p);
      }
      p++;
    }
    if (p >= end) return false;
    p++;
    if (out) *out = s;
    return true;
  }
  bool skip_value() {
    ws();
    if (p >= end) return false;
    if (*p == '"') return string(nullptr);
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      int depth = 0;
      while (p < end) {
        if (*p == '"') {
          if (!string(nullptr)) return false;
          continue;
        }
        if (*p == open) depth++;
        if (*p == close && --depth == 0) return p++, true;
        p++;
      }
      return false;
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']') p++;
    return true;
  }
};
}  // namespace

MER_EXPORT int mer_dataset_metadata_parse(const char *json, size_t len, mer_dataset_info *out) {
  if (!json || !out) return MER_ERR_INVALID_ARGUMENT;
  memset(out, 0, sizeof *out);
  out->dtype = -1;
  Json j{json, json + len};
  if (!j.lit('{')) return MER_ERR_VALIDATION_DISPATCH;
  if (j.lit('}')) return MER_OK;
  for (;;) {
    std::string key;
    if (!j.string(&key) || !j.lit(':')) return MER_ERR_VALIDATION_DISPATCH;
    j.ws();
    uint64_t *num = key == "format_version"          ? &out->format_version
                    : key == "num_experts"           ? &out->num_experts
                    : key == "d_model"               ? &out->d_model
                    : key == "d_ff"                  ? &out->d_ff
                    : key == "expert_size"           ? &out->expert_size
                    : key == "maximum_payload_bytes" ? &out->maximum_payload_bytes
                    : key == "block_align"           ? &out->block_align
                    : key == "experts_written"       ? &out->experts_written
                    : key == "num_layers"            ? &out->num_layers
                    : key == "experts_per_layer"     ? &out->experts_per_layer
                    : key == "top_k"                 ? &out->top_k
                                                     : nullptr;
    if (num && j.p < j.end && (isdigit((unsigned char)*j.p))) {
      char *e = nullptr;
      *num = strtoull(j.p, &e, 10);
      j.p = e;
      if (j.p < j.end && (*j.p == '.' || *j.p == 'e' || *j.p == 'E')) j.skip_value();  // a fraction: keep the integer part
    } else if (key == "dtype" || key == "q4_0_layout" || key == "conversion_mode") {
      std::string v;
      if (!j.string(&v)) return MER_ERR_VALIDATION_DISPATCH;
      if (key == "dtype") {
        snprintf(out->dtype_name, sizeof out->dtype_name, "%s", v.c_str());
        for (auto &c : v) c = (char)tolower((unsigned char)c);
        out->dtype = (v == "q4_0" || v == "q4-0") ? MER_DTYPE_Q4_0 : (v == "q8_0" || v == "q8-0") ? MER_DTYPE_Q8_0 : -1;
      } else if (key == "q4_0_layout") {
        snprintf(out->q4_0_layout, sizeof out->q4_0_layout, "%s", v.c_str());
      } else {
        snprintf(out->conversion_mode, sizeof out->conversion_mode, "%s", v.c_str());
      }
    } else if (!j.skip_value()) {
      return MER_ERR_VALIDATION_DISPATCH;
    }
    if (j.lit(',')) continue;
    if (j.lit('}')) return MER_OK;
    return MER_ERR_VALIDATION_DISPATCH;
  }
}
