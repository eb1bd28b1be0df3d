"""The allocation-free edge-attention entry point, called through its exported C symbol.

Some hosts of these kernels are not allowed to allocate device memory when they call in (a frozen memory pool,
a plugin that only receives pre-allocated tensors).  ``bf_edge_attn_fwd_noalloc`` serves them by keeping the
scratch of the long-row kernels in a fixed array inside the library.  The test drives it with ctypes exactly as
such a host would — raw pointers and a stream, no PyTorch binding — and compares with the regular entry point
and with the float32 PyTorch reference on two consecutive calls (the second call must not see the first call's
partial sums), checks that the call itself takes no device memory, and that bad arguments are refused on the host."""
import ctypes

import pytest
import torch

from budgetformer_b200.ops.edge_attention import edge_attention, edge_attention_reference
from tests.helpers import random_attn_graph

pytestmark = pytest.mark.gpu


class AttnParams(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("ldq", ctypes.c_longlong), ("ldk", ctypes.c_longlong), ("ldv", ctypes.c_longlong),
                ("out", ctypes.c_void_p), ("z", ctypes.c_void_p), ("rowptr", ctypes.c_void_p), ("col", ctypes.c_void_p),
                ("etype", ctypes.c_void_p), ("etab", ctypes.c_void_p),
                ("n", ctypes.c_int), ("hl", ctypes.c_int), ("hn", ctypes.c_int), ("dtype", ctypes.c_int),
                ("variant", ctypes.c_int), ("dropout_p", ctypes.c_float), ("dropout_seed", ctypes.c_uint32),
                ("hub_rows", ctypes.c_void_p), ("n_hub", ctypes.c_int), ("max_hub_degree", ctypes.c_int),
                ("hub_scratch", ctypes.c_void_p),
                ("out_dropout_p", ctypes.c_float), ("out_dropout_seed", ctypes.c_uint32),
                ("out_rows_local", ctypes.c_int), ("out_col0", ctypes.c_int)]


def _lib():
    from budgetformer_b200.ops import _ext
    mod = _ext.load()
    lib = ctypes.CDLL(mod.__file__)
    lib.bf_edge_attn_fwd_noalloc.argtypes = [ctypes.POINTER(AttnParams), ctypes.c_void_p]
    lib.bf_edge_attn_fwd_noalloc.restype = ctypes.c_int
    lib.bf_noalloc_strerror.argtypes = [ctypes.c_int]
    lib.bf_noalloc_strerror.restype = ctypes.c_char_p
    lib.bf_attn_params_size.argtypes = []
    lib.bf_attn_params_size.restype = ctypes.c_size_t
    # the structure above is a hand-written mirror of bf_attn_params: a silent drift of the layout would corrupt the call
    assert ctypes.sizeof(AttnParams) == lib.bf_attn_params_size(), (ctypes.sizeof(AttnParams), lib.bf_attn_params_size())
    return lib


def _call(lib, q, k, v, graph, hub_rows, max_deg, out=None, z=None, null_hub_rows=False, dtype_code=None):
    n, hl, hn = q.shape
    out = torch.empty_like(q) if out is None else out
    z = torch.empty(n, hl, dtype=torch.float32, device=q.device) if z is None else z
    p = AttnParams(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), ldq=q.stride(0), ldk=k.stride(0), ldv=v.stride(0),
                   out=out.data_ptr(), z=z.data_ptr(), rowptr=graph.rowptr.data_ptr(), col=graph.col.data_ptr(),
                   etype=None, etab=None, n=n, hl=hl, hn=hn,
                   dtype={torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[q.dtype] if dtype_code is None else dtype_code,
                   variant=0, dropout_p=0.0, dropout_seed=0,
                   hub_rows=hub_rows.data_ptr() if (hub_rows.numel() and not null_hub_rows) else None, n_hub=int(hub_rows.numel()),
                   max_hub_degree=int(max_deg), hub_scratch=None)
    rc = lib.bf_edge_attn_fwd_noalloc(ctypes.byref(p), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_entry_point_matches_regular_entry_point_twice(dtype):
    lib = _lib()
    dev = torch.device("cuda")
    n, hl, hn = 4500, 4, 16
    tol = 2e-4 if dtype == torch.float32 else 3e-2
    for call, (hub_row, seed) in enumerate([(6000, 1), (9000, 2)]):        # two calls in a row, different problems
        g = random_attn_graph(n, 9000, hub_row=hub_row, seed=seed).to(dev)
        deg = g.rowptr[1:] - g.rowptr[:-1]
        hubs = torch.nonzero(deg > 1024).flatten().to(torch.int32)
        assert hubs.numel() >= 1
        torch.manual_seed(seed)
        q, k, v = (torch.randn(n, hl, hn, device=dev).to(dtype) for _ in range(3))
        want = edge_attention(q, k, v, g)
        oracle = edge_attention_reference(q.float(), k.float(), v.float(), g)
        # outputs are allocated by the caller beforehand; the call itself must leave the device's free memory untouched
        out = torch.empty_like(q)
        z = torch.empty(n, hl, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc, got = _call(lib, q, k, v, g, hubs, int(deg.max()), out=out, z=z)
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info(dev)[0]
        assert rc == 0, lib.bf_noalloc_strerror(rc).decode()
        if call > 0:                                   # the first call on a device may load the module's image
            assert free_after == free_before, (free_before, free_after)
        scale = max(1.0, float(want.float().abs().max()))
        err = float((got.float() - want.float()).abs().max())
        assert err <= 2 * tol * scale, f"call {call}: max err {err} against the regular entry point"
        err = float((got.float() - oracle).abs().max())
        assert err <= 2 * tol * scale, f"call {call}: max err {err} against the float32 reference"


def test_noalloc_entry_point_rejects_oversized_problems():
    lib = _lib()
    dev = torch.device("cuda")
    g = random_attn_graph(64, 100, seed=0).to(dev)
    q = torch.zeros(64, 4, 16, device=dev)
    too_many = torch.zeros(65, dtype=torch.int32, device=dev)
    rc, _ = _call(lib, q, q, q, g, too_many, 2000)
    assert rc == -101 and b"exceeds" in lib.bf_noalloc_strerror(rc)
    wide = torch.zeros(64, 32, 64, device=dev)                             # 32 * 64 = 2048 > 1024 columns
    rc, _ = _call(lib, wide, wide, wide, g, torch.zeros(1, dtype=torch.int32, device=dev), 2000)
    assert rc == -101


def test_noalloc_entry_point_refuses_bad_arguments_on_the_host():
    """Rejected before anything is queued: nothing runs on the GPU, so nothing can fault."""
    lib = _lib()
    dev = torch.device("cuda")
    g = random_attn_graph(64, 100, seed=0).to(dev)
    q = torch.zeros(64, 4, 16, device=dev)
    one_hub = torch.zeros(1, dtype=torch.int32, device=dev)
    invalid = 1                                                            # cudaErrorInvalidValue
    rc, _ = _call(lib, q, q, q, g, one_hub, 2000, null_hub_rows=True)       # n_hub > 0 but no hub_rows
    assert rc == invalid
    rc, _ = _call(lib, q, q, q, g, one_hub, 0)                              # n_hub > 0 but no max_hub_degree
    assert rc == invalid
    rc, _ = _call(lib, q, q, q, g, one_hub, 2000, dtype_code=7)             # unknown dtype
    assert rc == invalid
    odd = torch.zeros(64, 4, 12, device=dev)                                # head size the kernels are not built for
    rc, _ = _call(lib, odd, odd, odd, g, one_hub, 2000)
    assert rc == invalid
