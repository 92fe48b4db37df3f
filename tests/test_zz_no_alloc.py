"""The no-allocation entry point (collected last on purpose: a run that stops at the first failure has
then already run every other test).

Some hosts cannot let a library call cudaMalloc for them - the device is fully owned by the host's
own pool and accounted byte by byte, or the call sits where cudaMalloc's device-wide synchronisation
is unacceptable.  mer_expert_forward_noalloc serves them from a fixed array inside the library.  Here
it is called through the C ABI twice in a row (the array keeps the first call's contents) and both
results are compared with the regular entry point and with the CPU oracle within the suite's FFN
tolerance; further cases check that the device's free memory does not move across calls, the largest
token count, and a second device when the machine has one."""
import ctypes

import numpy as np
import pytest

import mer_b200
import oracle

pytestmark = pytest.mark.gpu

FFN_TOL = 1e-3  # max-abs error relative to the RMS of the reference output, as in test_gpu_parity.py


def _rel(got, ref):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - ref)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30))


@pytest.mark.parametrize("dtype,D,F", [(mer_b200.DTYPE_Q4_0, 256, 512), (mer_b200.DTYPE_Q8_0, 128, 96)])
def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row(dtype, D, F):
    import torch
    synth = __import__("importlib").import_module("mer_b200.synth")
    torch.cuda.set_device(0)
    blob = synth.make_expert_blob(dtype, D, F, 77, 0, 0)
    xs = [synth.make_activations(5, D, 77, 0), synth.make_activations(3, D, 77, 1) * 3.0]
    stride = (256 + mer_b200.expert_bytes(dtype, D, F) + 4095) // 4096 * 4096
    with mer_b200.Backend(dtype, D, F, stride, 4, max_tokens=8) as b:
        b.admit(0, 1, blob)
        expected = [b.expert_forward_f32(0, 0, x) for x in xs]
    d_blob = torch.from_numpy(blob).cuda()
    stream = torch.cuda.current_stream().cuda_stream
    for x, ref in zip(xs, expected):  # two calls in a row on the shared scratch
        d_x = torch.from_numpy(x).cuda()
        d_out = torch.full((x.shape[0], D), float("nan"), device="cuda")
        mer_b200.expert_forward_noalloc(dtype, D, F, d_blob.data_ptr(), d_x.data_ptr(), x.shape[0], d_out.data_ptr(), 0.0, stream)
        torch.cuda.synchronize()
        got = d_out.cpu().numpy()
        for t in range(x.shape[0]):
            assert _rel(got[t], ref[t]) <= FFN_TOL
            assert _rel(got[t], oracle.expert_forward(dtype, blob, x[t], D, F)) <= FFN_TOL  # and against the CPU oracle


def test_noalloc_allocates_nothing_and_takes_the_largest_token_count():
    # the property the entry point exists for: after the first call (which looks the array's address up) the device's
    # free memory is the same before and after any number of calls; 8 tokens = MER_NOALLOC_MAX_TOKENS, two row passes
    import torch
    synth = __import__("importlib").import_module("mer_b200.synth")
    torch.cuda.set_device(0)
    dtype, D, F, n = mer_b200.DTYPE_Q8_0, 96, 160, 8
    blob = synth.make_expert_blob(dtype, D, F, 78, 0, 0)
    x = synth.make_activations(n, D, 78)
    d_blob, d_x = torch.from_numpy(blob).cuda(), torch.from_numpy(x).cuda()
    d_out = torch.empty(n, D, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    mer_b200.expert_forward_noalloc(dtype, D, F, d_blob.data_ptr(), d_x.data_ptr(), n, d_out.data_ptr(), 0.0, stream)  # warm-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        mer_b200.expert_forward_noalloc(dtype, D, F, d_blob.data_ptr(), d_x.data_ptr(), n, d_out.data_ptr(), 0.0, stream)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    got = d_out.cpu().numpy()
    for t in range(n):
        assert _rel(got[t], oracle.expert_forward(dtype, blob, x[t], D, F)) <= FFN_TOL


def test_noalloc_on_a_second_device():
    # the array's address is looked up once per device, with that device current
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    synth = __import__("importlib").import_module("mer_b200.synth")
    dtype, D, F, n = mer_b200.DTYPE_Q4_0, 64, 96, 3
    blob = synth.make_expert_blob(dtype, D, F, 79, 0, 0)
    x = synth.make_activations(n, D, 79)
    for dev in (1, 0, 1):
        torch.cuda.set_device(dev)
        d_blob, d_x = torch.from_numpy(blob).cuda(dev), torch.from_numpy(x).cuda(dev)
        d_out = torch.empty(n, D, device=f"cuda:{dev}")
        mer_b200.expert_forward_noalloc(dtype, D, F, d_blob.data_ptr(), d_x.data_ptr(), n, d_out.data_ptr(), 0.0,
                                        torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        got = d_out.cpu().numpy()
        for t in range(n):
            assert _rel(got[t], oracle.expert_forward(dtype, blob, x[t], D, F)) <= FFN_TOL
    torch.cuda.set_device(0)


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch():
    import torch
    torch.cuda.set_device(0)
    buf = torch.zeros(1024, device="cuda")
    with pytest.raises(mer_b200.GpuExpertDispatchError) as e:
        mer_b200.expert_forward_noalloc(mer_b200.DTYPE_Q8_0, 64, 64, buf.data_ptr(), buf.data_ptr(), 9, buf.data_ptr())
    assert e.value.kind == mer_b200.GpuExpertDispatchErrorKind.ValidationDispatch and "scratch" in e.value.detail
    with pytest.raises(mer_b200.GpuExpertDispatchError):
        mer_b200.expert_forward_noalloc(mer_b200.DTYPE_Q8_0, 64, 32768, buf.data_ptr(), buf.data_ptr(), 1, buf.data_ptr())
