"""The allocation-free MoE dispatch entry point (include/megray/no_alloc.h), called through its
exported C symbol, against the regular dispatch call on the same routing, twice in a row.

Why the entry point exists: some callers cannot allocate device memory at all (a server that
has given every free byte of HBM to its cache, a plugin that may not touch its host framework's
allocator, a loop that cannot afford cudaMalloc's implicit synchronisation).  For them the
per-expert cursors live in a fixed array inside the library.

Rows inside one expert's segment are handed out with atomics, so the two calls may place a token
on different rows; what must agree is the set of rows used per expert and the row contents each
(token, slot) finds at its recorded position.  This file sorts last so that a run that stops at
the first failure has already run every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(tokens=777, hidden=256, experts=8, seed=0):
    from megray_b200 import _lib

    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(seed)
    logits = torch.randn(tokens, experts, device="cuda", generator=g)
    src = torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16)
    idx = torch.empty(tokens, 2, dtype=torch.int32, device="cuda")
    w = torch.empty(tokens, 2, dtype=torch.float32, device="cuda")
    counts = torch.zeros(experts, dtype=torch.int32, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.megray_moe_route(logits.data_ptr(), tokens, experts, idx.data_ptr(), w.data_ptr(), counts.data_ptr(), st) == 0
    # one rank owns all experts: segments laid out back to back, padded to 128 rows
    padded = (counts + 127) // 128 * 128
    send_base = (torch.cumsum(padded, 0) - padded).to(torch.int32)
    capacity = int(padded.sum().item())
    return lib, st, src, idx, w, counts, send_base, capacity, tokens, hidden, experts


def _declare(lib):
    fn = lib.megray_moe_dispatch_noalloc
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                   C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_void_p]
    return fn


def test_no_alloc_dispatch_matches_the_regular_entry_point_twice():
    lib, st, src, idx, w, counts, send_base, capacity, T, H, E = _setup()
    noalloc = _declare(lib)
    for attempt in range(2):  # the built-in cursors keep the previous call's counts: must not matter
        use_w = attempt == 1
        wp = w.data_ptr() if use_w else None
        # regular entry point: caller-provided cursor array
        cursor = torch.zeros(E, dtype=torch.int32, device="cuda")
        dst_a = torch.zeros(capacity, H, dtype=torch.bfloat16, device="cuda")
        pos_a = torch.empty(T, 2, dtype=torch.int32, device="cuda")
        peers_a = (C.c_void_p * 1)(dst_a.data_ptr())
        assert lib.megray_moe_dispatch(src.data_ptr(), T, H, idx.data_ptr(), wp, send_base.data_ptr(),
                                       cursor.data_ptr(), None, pos_a.data_ptr(), peers_a, 1, E, capacity, st) == 0
        # allocation-free entry point
        dst_b = torch.zeros(capacity, H, dtype=torch.bfloat16, device="cuda")
        pos_b = torch.empty(T, 2, dtype=torch.int32, device="cuda")
        peers_b = (C.c_void_p * 1)(dst_b.data_ptr())
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]  # also sees a cudaMalloc made inside the library
        rc = noalloc(src.data_ptr(), T, H, idx.data_ptr(), wp, send_base.data_ptr(), E, pos_b.data_ptr(), peers_b, 1,
                     E, capacity, st)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        if attempt == 1:  # the first call on a device may load the kernel's module; later ones change nothing
            assert torch.cuda.mem_get_info()[0] >= free_before
        torch.cuda.synchronize()
        ia, ib = idx.flatten().long(), idx.flatten().long()
        pa, pb = pos_a.flatten().long(), pos_b.flatten().long()
        for e in range(E):
            ra = torch.sort(pa[ia == e]).values
            rb = torch.sort(pb[ib == e]).values
            assert torch.equal(ra, rb)  # the same rows of the expert's segment are in use
            lo = int(send_base[e].item())
            assert torch.equal(ra, torch.arange(lo, lo + int(counts[e].item()), device="cuda"))
        # every (token, slot) finds the same row contents at its recorded position
        got_a, got_b = dst_a[pa].float(), dst_b[pb].float()
        assert torch.allclose(got_a, got_b, rtol=0, atol=0)
        want = src.float().repeat_interleave(2, 0)
        if use_w:
            want = (want * w.flatten()[:, None]).to(torch.bfloat16).float()
        assert torch.allclose(got_b, want, rtol=2 ** -7, atol=1e-6)
        # rows that nobody owns stay untouched (zero)
        mask = torch.ones(capacity, dtype=torch.bool, device="cuda")
        mask[pb] = False
        assert float(dst_b[mask].abs().sum()) == 0.0


def test_no_alloc_dispatch_refuses_more_experts_than_its_array_holds():
    lib, st, src, idx, w, counts, send_base, capacity, T, H, E = _setup(tokens=64)
    noalloc = _declare(lib)
    pos = torch.empty(T, 2, dtype=torch.int32, device="cuda")
    dst = torch.zeros(capacity, H, dtype=torch.bfloat16, device="cuda")
    peers = (C.c_void_p * 1)(dst.data_ptr())
    rc = noalloc(src.data_ptr(), T, H, idx.data_ptr(), None, send_base.data_ptr(), 257, pos.data_ptr(), peers, 1, E,
                 capacity, st)
    assert rc == 6
    rc = noalloc(src.data_ptr(), T, H - 1, idx.data_ptr(), None, send_base.data_ptr(), E, pos.data_ptr(), peers, 1, E,
                 capacity, st)
    assert rc == 6
    torch.cuda.synchronize()
    assert float(dst.abs().sum()) == 0.0  # nothing was launched


def test_no_alloc_dispatch_drops_an_expert_id_nobody_owns():
    """A routing table with one expert id outside [0, experts): that (token, slot) is dropped
    (pos -1), every other row lands as usual, no other row of the buffer is touched.  The same
    table through the regular entry point behaves alike."""
    lib, st, src, idx, w, counts, send_base, capacity, T, H, E = _setup(tokens=200)
    noalloc = _declare(lib)
    bad = idx.clone()
    bad[17, 1] = E + 3          # beyond the experts of the call, inside the 256-entry array
    bad[42, 0] = -5
    for which in ("noalloc", "regular"):
        dst = torch.zeros(capacity + 128, H, dtype=torch.bfloat16, device="cuda")
        pos = torch.full((T, 2), -7, dtype=torch.int32, device="cuda")
        peers = (C.c_void_p * 1)(dst.data_ptr())
        if which == "noalloc":
            rc = noalloc(src.data_ptr(), T, H, bad.data_ptr(), None, send_base.data_ptr(), E, pos.data_ptr(), peers,
                         1, E, capacity, st)
        else:
            cursor = torch.zeros(E, dtype=torch.int32, device="cuda")
            rc = lib.megray_moe_dispatch(src.data_ptr(), T, H, bad.data_ptr(), None, send_base.data_ptr(),
                                         cursor.data_ptr(), None, pos.data_ptr(), peers, 1, E, capacity, st)
        assert rc == 0
        torch.cuda.synchronize()
        p = pos.flatten().long()
        valid = ((bad.flatten() >= 0) & (bad.flatten() < E))
        assert int((~valid).sum()) == 2
        assert bool((p[~valid] == -1).all())
        assert bool((p[valid] >= 0).all()) and bool((p[valid] < capacity).all())
        assert p[valid].unique().numel() == int(valid.sum())          # every kept pair has a row of its own
        want = src.float().repeat_interleave(2, 0)[valid]
        assert torch.equal(dst[p[valid]].float(), want)
        mask = torch.ones(capacity + 128, dtype=torch.bool, device="cuda")
        mask[p[valid]] = False
        assert float(dst[mask].abs().sum()) == 0.0                    # nothing else was written
    # more experts than the given owners can hold: refused
    pos = torch.empty(T, 2, dtype=torch.int32, device="cuda")
    dst = torch.zeros(capacity, H, dtype=torch.bfloat16, device="cuda")
    peers = (C.c_void_p * 1)(dst.data_ptr())
    assert noalloc(src.data_ptr(), T, H, idx.data_ptr(), None, send_base.data_ptr(), E, pos.data_ptr(), peers, 1,
                   E - 1, capacity, st) == 6
