"""``omnikv_decode_attn_no_alloc``: the decode-attention entry point for callers that cannot allocate.

Some users of the library are handed tensors but no allocator (an operator plugged into a runtime that owns
all device memory, a process with a fixed memory budget, a loop that must never call ``cudaMalloc``).  For them the split partials
live in a fixed 4 MiB array inside the library.  This file checks that entry point against the regular one
(``omnikv_decode_attn``, caller-owned workspace) through the C ABI, twice in a row -- the array is shared by
all calls and keeps the previous call's contents, so the second call must not be disturbed by the first --
and that a problem larger than the array is refused.  It is named to be collected last.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-4)])
def test_no_alloc_matches_regular_entry_point_twice(dtype, tol):
    from omnikv_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    B, H, KVH, d = 2, 32, 8, 128
    for call, (L, k_sel, tail, splits) in enumerate([(6000, 402, 3, 9), (3000, 0, 0, 4)]):
        # first a sparse-layer shape (selected rows + tail), then a dense one with other sizes, back to back
        kc = torch.randn(B, KVH, L + 8, d, generator=g, device="cuda").to(dtype)
        vc = torch.randn(B, KVH, L + 8, d, generator=g, device="cuda").to(dtype)
        q = (torch.randn(B, H, d, generator=g, device="cuda") * 1.5).to(dtype)
        if k_sel:
            idx = torch.stack([torch.sort(torch.randperm(L, generator=g, device="cuda")[:k_sel]).values for _ in range(B)])
            kw = dict(idx=idx.to(torch.int32).contiguous(), k_tail=kc, v_tail=vc, tail_start=_i32([L] * B),
                      tail_len=_i32([tail, tail - 1]))
            len_a = _i32([k_sel, k_sel - 7])
        else:
            kw, len_a = {}, _i32([L, L - 999])
        want = ops.decode_attn(q, kc, vc, len_a, n_splits=splits, **kw)
        got = torch.full_like(q, float("nan"))
        ops.decode_attn_no_alloc(q, kc, vc, len_a, got, n_splits=splits, **kw)
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        assert err <= tol, (call, err)
        assert torch.equal(got, want)  # same kernel, same split plan: the results are in fact identical


def test_no_alloc_refuses_what_does_not_fit():
    import ctypes

    from omnikv_b200 import abi, ops
    B, H, KVH, d = 8, 32, 8, 128
    q = torch.zeros(B, H, d, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(B, KVH, 64, d, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(q)
    with pytest.raises(abi.OmniKVError, match="built-in scratch"):
        ops.decode_attn_no_alloc(q, kc, kc, _i32([64] * B), out, n_splits=64)  # 8*32*64 = 16384 > 8034
    # the C entry point itself refuses too, before launching anything
    p = abi.AttnParams()
    p.dtype, p.B, p.H, p.KVH, p.head_dim, p.n_splits = abi.BF16, B, H, KVH, d, 64
    p.q, p.out, p.kA, p.vA, p.lenA = q.data_ptr(), out.data_ptr(), kc.data_ptr(), kc.data_ptr(), _i32([64] * B).data_ptr()
    assert abi.lib().omnikv_decode_attn_no_alloc(ctypes.byref(p), None) == -3


def test_no_alloc_first_call_then_graph_replay():
    """The documented order of use: the first call on a device (which looks up the built-in array's address) is made
    outside stream capture; after that the entry point is captured and replayed like any other launch, and the
    replays -- over changing inputs -- equal the regular entry point."""
    from omnikv_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(5)
    B, H, KVH, d, L, splits = 1, 32, 8, 128, 4096, 8
    kc = torch.randn(B, KVH, L, d, generator=g, device="cuda").to(torch.bfloat16)
    vc = torch.randn(B, KVH, L, d, generator=g, device="cuda").to(torch.bfloat16)
    q = torch.randn(B, H, d, generator=g, device="cuda").to(torch.bfloat16)
    n = _i32([L])
    out = torch.empty_like(q)
    ops.decode_attn_no_alloc(q, kc, vc, n, out, n_splits=splits)  # first call: outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.decode_attn_no_alloc(q, kc, vc, n, out, n_splits=splits)
    for rep in range(3):
        q.copy_(torch.randn(B, H, d, generator=g, device="cuda").to(torch.bfloat16))
        n.fill_(L - 100 * rep)
        graph.replay()
        want = ops.decode_attn(q, kc, vc, n, n_splits=splits)
        torch.cuda.synchronize()
        assert torch.equal(out, want), rep
