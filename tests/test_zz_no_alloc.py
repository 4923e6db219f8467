"""px_triangle_multiplication_static: the tri-mul entry point for callers that cannot allocate.

Some hosts of this library have no way to give it a workspace: a plug-in inside an application
that has already handed every byte of device memory to its own pool (cudaMalloc fails there), or a
latency-critical thread that may not call cudaMalloc/cudaFree because those synchronise the whole
device.  For them the library carries a fixed 16 MiB scratch array in its own image (N <= 128).
This test drives that entry point through the C ABI and compares it with the workspace-taking
entry point on the same inputs, twice in a row with different sizes, because the second call finds
the first call's leftovers in the shared array.

Collected last on purpose (file name): a failure here cannot hide the other tests' results.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-2  # the tolerance of the other GPU parity tests (relative Frobenius error)


def _relf(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def _args(n, seed, zdtype):
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(n, n, 128, generator=g).to(zdtype).cuda()
    mask = (torch.rand(n, n, generator=g) > 0.15).float().cuda()
    vec = lambda s: (s * torch.randn(128, generator=g)).cuda()
    ln = [1 + vec(0.1), vec(0.1), 1 + vec(0.1), vec(0.1)]
    # 16-bit weights as the C ABI wants them: in the format of the rows they multiply (bf16 rows as stored, fp32 rows
    # as fp16), except w_z (index 4), which multiplies the fp16 intermediate x
    zfmt = torch.bfloat16 if zdtype == torch.bfloat16 else torch.float16
    ws = [(torch.randn(128, 128, generator=g) / 128 ** 0.5).to(torch.float16 if i == 4 else zfmt).cuda() for i in range(6)]
    return z, mask, ln, ws


def _oracle_update(n, seed, zdtype, incoming):
    """The same update from the CPU oracle (fp32), fed with the tensors _args draws."""
    from oracle import pairformer_oracle as O

    z, mask, ln, ws = _args(n, seed, zdtype)
    keys = ("linear_a_p", "linear_a_g", "linear_b_p", "linear_b_g", "linear_z", "linear_g")
    p = {f"{k}.weight": w.float().cpu() for k, w in zip(keys, ws)}
    p.update({"layer_norm_in.weight": ln[0].cpu(), "layer_norm_in.bias": ln[1].cpu(),
              "layer_norm_out.weight": ln[2].cpu(), "layer_norm_out.bias": ln[3].cpu()})
    return O.triangle_multiplication(z.float().cpu(), mask.cpu(), p, outgoing=not incoming)


def _run(lib, static, n, seed, zdtype, incoming):
    from protenix_b200 import _lib

    z, mask, ln, ws = _args(n, seed, zdtype)
    out = torch.full_like(z, float("nan"))
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    st = torch.cuda.current_stream().cuda_stream
    dt = _lib.PX_BF16 if zdtype == torch.bfloat16 else _lib.PX_F32
    common = [P(z), P(out), dt, P(mask)] + [P(t) for t in ln] + [P(w) for w in ws]
    if static:
        rc = lib.px_triangle_multiplication_static(*common, n, int(incoming), 1, 1e-5, st)
    else:
        nbytes = lib.px_trimul_workspace_bytes(n)
        work = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        rc = lib.px_triangle_multiplication(*common, P(work), nbytes, n, int(incoming), 1, 1e-5, st)
    torch.cuda.synchronize()
    assert rc == 0, lib.px_status_string(rc)
    return out, z


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from protenix_b200 import _lib

    lib = _lib.load()
    assert lib.px_static_max_n() == 128
    # two calls in a row: a large N first, then a smaller N with another layout of the same array,
    # then the large one again with the other direction and storage type
    for n, seed, zdtype, incoming in ((128, 1, torch.bfloat16, False), (52, 2, torch.float32, True),
                                      (101, 3, torch.bfloat16, True)):
        got, z = _run(lib, True, n, seed, zdtype, incoming)
        want, _ = _run(lib, False, n, seed, zdtype, incoming)
        assert torch.isfinite(got.float()).all()
        assert _relf(got, want) <= TOL, (n, _relf(got, want))
        assert torch.equal(got, want), "same kernels on the same inputs must give the same bits"
        assert _relf(got.float() - z.float(), want.float() - z.float()) <= TOL   # the update itself, not z + update
        upd = _oracle_update(n, seed, zdtype, incoming)
        assert _relf(got.float().cpu() - z.float().cpu(), upd) <= TOL, "against the CPU oracle, not only its sibling"


def test_static_scratch_rejects_sizes_beyond_its_capacity():
    from protenix_b200 import _lib

    lib = _lib.load()
    z, mask, ln, ws = _args(16, 0, torch.bfloat16)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    common = [P(z), P(z), _lib.PX_BF16, P(mask)] + [P(t) for t in ln] + [P(w) for w in ws]
    rc = lib.px_triangle_multiplication_static(*common, 129, 0, 1, 1e-5, None)
    assert rc == -5 and b"built-in scratch" in lib.px_status_string(rc)
    assert lib.px_triangle_multiplication_static(*common, 0, 0, 1, 1e-5, None) == -1
