"""On-disk formats around the expert path: Unified Tensor Header (tensor_header.rs) and metadata.json
(main.rs:9096-9114), parsed by the library; the file loader mer_expert_admit_file on a GPU."""
import importlib
import json
import os
import struct

import numpy as np
import pytest

import mer_b200
import oracle

formats = importlib.import_module("mer_b200.formats")
synth = importlib.import_module("mer_b200.synth")


def test_uth1_header_layout_and_roundtrip():
    # roundtrip_swiglu_header / writer layout (tensor_header.rs:9-27, 419-499, 569-586)
    for dtype, uth_id in ((mer_b200.DTYPE_Q4_0, 4), (mer_b200.DTYPE_Q8_0, 5)):
        h = formats.uth1_header(dtype, 512, 2048, block_align=4096)
        assert h.size == 4096 and bytes(h[:4]) == b"UTH1"
        version, dt, rank = struct.unpack_from("<HBB", h, 4)
        assert (version, dt, rank) == (1, uth_id, 3)
        assert struct.unpack_from("<4I", h, 8) == (2048, 512, 3, 0)  # [d_ff, d_model, 3]
        assert struct.unpack_from("<2I", h, 24) == (0, 0)            # no global scale region for block formats
        assert struct.unpack_from("<3I", h, 32) == (16, 16, 64)
        assert struct.unpack_from("<I", h, 44) == (1,)               # payload is page aligned
        assert not h[48:].any()
        info, payload = formats.uth_probe(np.concatenate([h, np.arange(100, dtype=np.uint8)]))
        assert (info["kind"], info["version"], info["dtype"], info["d_model"], info["d_ff"]) == (1, 1, dtype, 512, 2048)
        assert info["payload_offset"] == 4096 and payload.tolist() == list(range(100))
    # block_align 0: the payload starts right after the 64 bytes (tensor_header.rs:524-527)
    h = formats.uth1_header(mer_b200.DTYPE_Q8_0, 64, 96, block_align=4096)
    info, payload = formats.uth_probe(h, block_align=0)
    assert info["payload_offset"] == 64 and payload.size == 4096 - 64


def test_blobs_without_a_valid_header_are_legacy_blobs():
    # strip returns the bytes unchanged for a missing magic, a short buffer, version 0 or too new, rank 0 or > 4,
    # an unknown dtype id, and a header whose padding runs past the buffer (tensor_header.rs:501-545)
    good = formats.uth1_header(mer_b200.DTYPE_Q4_0, 32, 64)
    cases = [np.zeros(4096, np.uint8), good[:63]]
    for off, val in ((4, 0), (4, 2), (7, 0), (7, 5), (6, 11)):
        bad = good.copy()
        bad[off] = val
        cases.append(bad)
    cases.append(good[:100])  # flag says page aligned, but the buffer ends before the payload
    for c in cases:
        info, payload = formats.uth_probe(c)
        assert info["kind"] == 0 and info["payload_offset"] == 0 and payload.size == c.size
    info, _ = formats.uth_probe(good)
    assert info["kind"] == 1
    f32 = good.copy()
    f32[6] = 0  # a dtype this library does not run is still a valid header
    info, _ = formats.uth_probe(f32)
    assert info["kind"] == 1 and info["dtype"] == -1 and info["uth_dtype_id"] == 0


def test_uth2_mixed_header_roundtrip_and_validation():
    # MixedExpertHeader::to_bytes / probe / validate / strip (tensor_header.rs:195-391)
    ranges = [(5, 0, 16, 4), (5, 16, 16, 4), (5, 32, 16, 4)]
    h = formats.uth2_header(2, 2, ranges, block_align=8192)
    assert h.size == 8192 and bytes(h[:4]) == b"UTH2"
    assert struct.unpack_from("<HH", h, 4) == (2, 3)
    assert struct.unpack_from("<3I", h, 8) == (2, 2, 1)
    for i, (dt, off, ln, w) in enumerate(ranges):
        base = 24 + 24 * i
        assert (h[base], h[base + 1]) == (dt, i)
        assert struct.unpack_from("<QQI", h, base + 4) == (off, ln, w)
    blob = np.concatenate([h, np.full(64, 0x5A, np.uint8)])
    info, payload = formats.uth_probe(blob, block_align=8192)
    assert info["kind"] == 2 and info["dtype"] == mer_b200.DTYPE_Q8_0 and (info["d_model"], info["d_ff"]) == (2, 2)
    assert [(p["offset"], p["len"], p["weights"]) for p in info["proj"]] == [(0, 16, 4), (16, 16, 4), (32, 16, 4)]
    assert payload.size == 64 and (payload == 0x5A).all()
    mixed = formats.uth2_header(2, 2, [(4, 0, 16, 4), (5, 16, 16, 4), (5, 32, 16, 4)], block_align=8192)
    info, _ = formats.uth_probe(np.concatenate([mixed, np.zeros(64, np.uint8)]), block_align=8192)
    assert info["kind"] == 2 and info["dtype"] == -1  # projections of different dtypes: valid, but not runnable here
    # invalid: overlapping ranges, a range past the payload, a zero-length range, wrong role byte, zero shape
    for bad_ranges in ([(5, 0, 16, 4), (5, 8, 16, 4), (5, 32, 16, 4)], [(5, 0, 16, 4), (5, 16, 16, 4), (5, 60, 16, 4)],
                       [(5, 0, 0, 4), (5, 16, 16, 4), (5, 32, 16, 4)], [(10, 0, 16, 4), (5, 16, 16, 4), (5, 32, 16, 4)]):
        b = np.concatenate([formats.uth2_header(2, 2, bad_ranges, block_align=8192), np.zeros(64, np.uint8)])
        assert formats.uth_probe(b, block_align=8192)[0]["kind"] == 0
    swapped = blob.copy()
    swapped[24 + 1], swapped[48 + 1] = 1, 0
    assert formats.uth_probe(swapped, block_align=8192)[0]["kind"] == 0
    zero = np.concatenate([formats.uth2_header(0, 2, ranges, block_align=8192), np.zeros(64, np.uint8)])
    assert formats.uth_probe(zero, block_align=8192)[0]["kind"] == 0


def test_metadata_json_is_parsed_with_unknown_keys_skipped():
    meta = {"format_version": 2, "conversion_mode": "synthetic", "num_experts": 256, "d_model": 4096, "d_ff": 14336,
            "expert_size": 99094528, "maximum_payload_bytes": 99090432, "block_align": 4096, "dtype": "q4_0",
            "weight_layout": "gate_proj || up_proj || down_proj (row-major)", "q4_0_layout": "ggml-standard-v1",
            "experts_written": 256, "nested": {"a": [1, 2, {"b": "}"}], "s": 'x"y'}, "ratio": 0.5, "flag": True, "none": None}
    got = formats.parse_metadata(json.dumps(meta, indent=2) + "\n")
    for k in ("format_version", "num_experts", "d_model", "d_ff", "expert_size", "maximum_payload_bytes", "block_align", "experts_written"):
        assert got[k] == meta[k], k
    assert got["dtype"] == mer_b200.DTYPE_Q4_0 and got["dtype_name"] == "q4_0" and got["q4_0_layout"] == "ggml-standard-v1"
    assert got["conversion_mode"] == "synthetic"
    assert formats.parse_metadata('{"dtype": "q8_0", "d_model": 2048}')["dtype"] == mer_b200.DTYPE_Q8_0
    assert formats.parse_metadata('{"dtype": "f32"}')["dtype"] == -1
    assert formats.parse_metadata("{}")["num_experts"] == 0
    for bad in ("", "[1, 2]", '{"d_model" 4}', '{"dtype": "q4_0"'):
        with pytest.raises(ValueError):
            formats.parse_metadata(bad)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,D,F", [(oracle.Q4_0, 256, 512), (oracle.Q8_0, 64, 96)])
def test_expert_files_load_into_hbm_slots(tmp_path, dtype, D, F):
    # gen-data style dataset: expert_<id>.bin with a page-padded UTH1 header (and one legacy file without), metadata.json
    blobs = [synth.make_expert_blob(dtype, D, F, 77, 0, e) for e in range(3)]
    meta = formats.write_dataset(str(tmp_path), dtype, D, F, blobs)
    parsed = formats.parse_metadata(open(tmp_path / "metadata.json").read())
    assert (parsed["d_model"], parsed["d_ff"], parsed["dtype"], parsed["num_experts"]) == (D, F, dtype, 3)
    assert parsed["expert_size"] % parsed["block_align"] == 0 and parsed["expert_size"] == meta["expert_size"]
    legacy = tmp_path / "expert_legacy.bin"
    blobs[1].tofile(legacy)
    # a UTH2 file whose three projections sit in reverse order inside the payload
    proj = blobs[2].size // 3
    pay = np.concatenate([blobs[2][2 * proj:], blobs[2][proj:2 * proj], blobs[2][:proj]])
    uid = 4 if dtype == oracle.Q4_0 else 5
    h2 = formats.uth2_header(D, F, [(uid, 2 * proj, proj, D * F), (uid, proj, proj, D * F), (uid, 0, proj, D * F)])
    mixed = tmp_path / "expert_mixed.bin"
    np.concatenate([h2, pay]).tofile(mixed)
    x = synth.make_activations(2, D, 77)
    stride = (256 + mer_b200.expert_bytes(dtype, D, F) + 4095) // 4096 * 4096
    with mer_b200.Backend(dtype, D, F, stride * 4, 16, max_tokens=4) as b:
        b.admit_file(0, 1, str(tmp_path / "expert_0.bin"), parsed["block_align"])
        b.admit_file(1, 1, str(legacy), parsed["block_align"])
        b.admit_file(2, 1, str(mixed), parsed["block_align"], wait=False)
        for e in range(3):
            got = b.expert_forward_f32(0, e, x)
            ref = oracle.expert_forward(dtype, blobs[e], x[0], D, F)
            assert float(np.abs(got[0] - ref).max() / np.sqrt(np.mean(ref.astype(np.float64) ** 2))) <= 1e-3
            projb = oracle.projection_bytes(dtype, D, F)
            deq = b.dequant_projection(e, 2)
            assert (deq.view(np.uint32) == oracle.dequant_stream(dtype, blobs[e][2 * projb:], D * F).view(np.uint32)).all()
        # typed failures: a truncated file, a wrong shape, a wrong dtype, a missing file
        short = tmp_path / "short.bin"
        np.fromfile(tmp_path / "expert_0.bin", dtype=np.uint8)[:4096 + 100].tofile(short)
        other = tmp_path / "other_shape.bin"
        np.concatenate([formats.uth1_header(dtype, D, F + 32), blobs[0]]).tofile(other)
        wrong = tmp_path / "other_dtype.bin"
        np.concatenate([formats.uth1_header(1 - dtype, D, F), blobs[0]]).tofile(wrong)
        for path, kind in ((short, "Upload"), (other, "ValidationDispatch"), (wrong, "ValidationDispatch"),
                           (tmp_path / "missing.bin", "Upload")):
            with pytest.raises(mer_b200.GpuExpertDispatchError) as err:
                b.admit_file(5, 1, str(path), 4096)
            assert err.value.kind.name == kind, path
        assert not b.contains_generation(5, 1)
