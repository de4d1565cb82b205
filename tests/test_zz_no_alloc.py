"""The allocation-free attention entry point (b200dec_attention_static) against the regular one.

It exists for hosts that may not allocate device memory where they call the library (a memory pool frozen at start-up,
a plugin interface that passes only inputs and outputs, a foreign-language runtime that would not see the allocation):
its split workspace is an array inside the library. Here it is called through the C-ABI twice in a row on different
inputs (the array keeps the previous call's contents) and must give exactly the regular entry point's output, which
runs the same kernel with a caller-owned workspace. The file name sorts last so that a run that stops at the first
failure has already run every other test."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, rows, H, D, S, cap, self_):
    rng = np.random.default_rng(seed)
    dev = "cuda"
    kc = torch.from_numpy(rng.standard_normal((S + 1, H, cap, D)).astype(np.float32)).to(dev).to(torch.bfloat16)
    vc = torch.from_numpy(rng.standard_normal((S + 1, H, cap, D)).astype(np.float32)).to(dev).to(torch.bfloat16)
    active = torch.from_numpy(rng.permutation(S)[:rows].astype(np.int32)).to(dev)
    n = torch.from_numpy(rng.integers(1, cap - 1, S + 1).astype(np.int32)).to(dev)
    q = torch.from_numpy(rng.standard_normal((rows, (3 if self_ else 1) * H * D)).astype(np.float32)).to(dev)
    return kc, vc, active, n, q


@pytest.mark.parametrize("H,D,self_", [(16, 64, 0), (16, 64, 1), (8, 128, 0)])
def test_static_workspace_matches_caller_workspace(H, D, self_):
    from cohere_inference_b200 import native as nv
    lib = nv.lib()
    rows, S, cap = 5, 8, 300  # few rows: every row is split into spans, so the workspace is really used
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call in range(2):  # two calls in a row: the second finds the first one's leftovers in the array
        kc, vc, active, n, q = _inputs(100 + call, rows, H, D, S, cap, self_)
        ld = q.shape[1]
        outs = []
        for static in (False, True):
            k2, v2 = kc.clone(), vc.clone()  # self-attention appends into the cache
            out = torch.zeros(rows, H * D, device="cuda")
            if static:
                nv.check(lib.b200dec_attention_static(self_, nv.ptr(active), nv.ptr(q), ld, nv.ptr(k2), nv.ptr(v2),
                                                      nv.ptr(n), S, H, D, cap, D ** -0.5, nv.ptr(out), nv.OUT_F32, rows,
                                                      nv.ptr(status), 0, nv.stream_ptr()))
            else:
                part = torch.zeros(lib.b200dec_attention_scratch_floats(rows, H, D), device="cuda")
                count = torch.zeros(rows * H, dtype=torch.int32, device="cuda")
                nv.check(lib.b200dec_attention(self_, nv.ptr(active), nv.ptr(q), ld, nv.ptr(k2), nv.ptr(v2), nv.ptr(n), S,
                                               H, D, cap, D ** -0.5, nv.ptr(out), nv.OUT_F32, rows, nv.ptr(part),
                                               nv.ptr(count), nv.ptr(status), 0, nv.stream_ptr()))
            torch.cuda.synchronize()
            outs.append((out.cpu().numpy(), k2.float().cpu().numpy(), v2.float().cpu().numpy()))
        # same kernel, same span order: bit-identical output and cache (the tolerance of the other attention tests,
        # 2e-5, would also hold; equality is the stronger statement)
        for a, b in zip(outs[0], outs[1]):
            assert np.array_equal(a, b)
        assert np.isfinite(outs[1][0]).all() and np.abs(outs[1][0]).max() > 0
    assert int(status.item()) == 0


def test_static_workspace_refuses_sizes_beyond_its_capacity():
    from cohere_inference_b200 import native as nv
    lib = nv.lib()
    kc, vc, active, n, q = _inputs(7, 4, 16, 64, 4, 64, 0)
    out = torch.zeros(64, 1024, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.b200dec_attention_static(0, nv.ptr(active), nv.ptr(q), 1024, nv.ptr(kc), nv.ptr(vc), nv.ptr(n), 4, 16, 64, 64,
                                      0.125, nv.ptr(out), nv.OUT_F32, 64, nv.ptr(status), 0, nv.stream_ptr())
    assert rc == 1 and b"exceeds the built-in workspace" in lib.b200dec_last_error()
    torch.cuda.synchronize()


def test_static_call_captured_into_a_graph_and_replayed():
    """After its first (set-up) call the entry point is two stream operations, a memset of the arrival counters and the
    kernel: captured into a CUDA graph with the programmatic-launch flag set (which the entry point ignores, its
    kernel follows a memset) and replayed twice on changed inputs, it gives the regular entry point's bits each time."""
    from cohere_inference_b200 import native as nv
    lib = nv.lib()
    H, D, self_, rows, S, cap = 16, 64, 1, 5, 8, 300
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kc, vc, active, n, q = _inputs(200, rows, H, D, S, cap, self_)
    ld = q.shape[1]
    out = torch.zeros(rows, H * D, device="cuda")
    k2, v2 = kc.clone(), vc.clone()

    def static_call():
        nv.check(lib.b200dec_attention_static(self_, nv.ptr(active), nv.ptr(q), ld, nv.ptr(k2), nv.ptr(v2), nv.ptr(n), S, H,
                                              D, cap, D ** -0.5, nv.ptr(out), nv.OUT_F32, rows, nv.ptr(status), 1,
                                              nv.stream_ptr()))
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        static_call()  # the set-up call: looks the array's address up, outside any capture
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        static_call()
    for replay in range(2):
        kc_r, vc_r, active_r, n_r, q_r = _inputs(300 + replay, rows, H, D, S, cap, self_)
        for dst, src in ((k2, kc_r), (v2, vc_r), (active, active_r), (n, n_r), (q, q_r)):
            dst.copy_(src)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        k3, v3 = kc_r.clone(), vc_r.clone()
        want = torch.zeros(rows, H * D, device="cuda")
        part = torch.zeros(lib.b200dec_attention_scratch_floats(rows, H, D), device="cuda")
        count = torch.zeros(rows * H, dtype=torch.int32, device="cuda")
        nv.check(lib.b200dec_attention(self_, nv.ptr(active_r), nv.ptr(q_r), ld, nv.ptr(k3), nv.ptr(v3), nv.ptr(n_r), S, H,
                                       D, cap, D ** -0.5, nv.ptr(want), nv.OUT_F32, rows, nv.ptr(part), nv.ptr(count),
                                       nv.ptr(status), 0, nv.stream_ptr()))
        torch.cuda.synchronize()
        assert torch.equal(out, want) and torch.equal(k2, k3) and torch.equal(v2, v3)
        assert float(out.abs().max()) > 0
    assert int(status.item()) == 0
