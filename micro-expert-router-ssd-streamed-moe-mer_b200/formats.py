"""Mirror of the reference's on-disk formats around the expert path over the C ABI: the Unified Tensor Header
(tensor_header.rs: TensorHeader / MixedExpertHeader) and a dataset's metadata.json (main.rs:9096-9114)."""
import ctypes as C
import json
import os

import numpy as np

from . import capi

UTH_DTYPE_Q4_0, UTH_DTYPE_Q8_0 = 4, 5


def uth_probe(data, block_align=4096):
    """TensorHeader::strip / MixedExpertHeader::strip: returns (info dict, payload view).  A blob without a valid
    header comes back unchanged with kind 0."""
    buf = np.ascontiguousarray(np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data, dtype=np.uint8)
    info = capi.MerUthInfo()
    rc = capi.load_library().mer_uth_probe(buf.ctypes.data_as(C.c_void_p), buf.size, block_align, C.byref(info))
    assert rc == 0
    d = {"kind": info.kind, "version": info.version, "uth_dtype_id": info.uth_dtype_id, "dtype": info.dtype,
         "shape": list(info.shape)[:info.shape_rank], "flags": info.flags, "d_model": info.d_model, "d_ff": info.d_ff,
         "payload_offset": info.payload_offset, "payload_bytes": info.payload_bytes,
         "proj": [{"uth_dtype_id": p.uth_dtype_id, "weights": p.weights, "offset": p.offset, "len": p.len} for p in info.proj]}
    return d, buf[info.payload_offset:]


def uth1_header(dtype, d_model, d_ff, block_align=4096):
    """TensorHeader::for_swiglu_expert(...).write_padded(block_align): header bytes + zero padding."""
    lib = capi.load_library()
    n = C.c_size_t(0)
    out = np.zeros(max(block_align, 64) + 64, np.uint8)
    rc = lib.mer_uth1_write(dtype, d_model, d_ff, block_align, out.ctypes.data_as(C.c_void_p), out.size, C.byref(n))
    assert rc == 0
    return out[:n.value].copy()


def uth2_header(d_model, d_ff, ranges, block_align=4096):
    """MixedExpertHeader::new(d_model, d_ff, gate, up, down).write_padded(block_align); ranges = 3 x (dtype id, offset,
    len, weights) relative to the payload."""
    lib = capi.load_library()
    arr = (capi.MerUthProjection * 3)(*[capi.MerUthProjection(r[0], r[3], r[1], r[2]) for r in ranges])
    n = C.c_size_t(0)
    out = np.zeros(max(block_align, 128) + 128, np.uint8)
    rc = lib.mer_uth2_write(d_model, d_ff, arr, block_align, out.ctypes.data_as(C.c_void_p), out.size, C.byref(n))
    assert rc == 0
    return out[:n.value].copy()


def parse_metadata(text):
    info = capi.MerDatasetInfo()
    raw = text.encode() if isinstance(text, str) else bytes(text)
    rc = capi.load_library().mer_dataset_metadata_parse(raw, len(raw), C.byref(info))
    if rc != 0:
        raise ValueError("metadata.json is not a JSON object this loader understands")
    d = {n: int(getattr(info, n)) for n, _ in info._fields_[:11]}
    d.update(dtype=info.dtype, dtype_name=info.dtype_name.decode(), q4_0_layout=info.q4_0_layout.decode(),
             conversion_mode=info.conversion_mode.decode())
    return d


def write_dataset(data_dir, dtype, d_model, d_ff, blobs, block_align=4096, header="uth1"):
    """Writes expert_<id>.bin files (optionally with a UTH1 header, page padded as gguf-convert does) and the
    metadata.json of main.rs:9096-9114.  For tests and examples."""
    os.makedirs(data_dir, exist_ok=True)
    payload = max(len(b) for b in blobs)
    hdr = uth1_header(dtype, d_model, d_ff, block_align) if header == "uth1" else np.zeros(0, np.uint8)
    expert_size = (len(hdr) + payload + block_align - 1) // block_align * block_align
    for i, blob in enumerate(blobs):
        body = np.zeros(expert_size, np.uint8)
        body[:len(hdr)] = hdr
        body[len(hdr):len(hdr) + len(blob)] = blob
        body.tofile(os.path.join(data_dir, f"expert_{i}.bin"))
    meta = {"format_version": 2, "conversion_mode": "synthetic", "num_experts": len(blobs), "d_model": d_model, "d_ff": d_ff,
            "expert_size": expert_size, "maximum_payload_bytes": payload, "block_align": block_align,
            "dtype": "q4_0" if dtype == capi.DTYPE_Q4_0 else "q8_0",
            "weight_layout": "gate_proj || up_proj || down_proj (row-major)", "q4_0_layout": "ggml-standard-v1",
            "experts_written": len(blobs)}
    with open(os.path.join(data_dir, "metadata.json"), "w") as f:
        f.write(json.dumps(meta, indent=2) + "\n")
    return meta
