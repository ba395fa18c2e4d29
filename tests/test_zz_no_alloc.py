"""fbb_flash64_f16_static: flash attention whose scratch memory is a device array inside the library.

The file name sorts last on purpose: the entry point shares one array between all calls of the process, so it is
exercised after everything else has run (and the tests also pass when this file is run alone).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(fn_name, q, k, v, out, variant, *extra):
    from fastbb_b200 import _lib
    B, N, H, _ = q.shape
    lib = _lib.load()
    _lib.check(getattr(lib, fn_name)(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), B, N, H, *q.stride()[:3], *k.stride()[:3],
                                     *v.stride()[:3], *out.stride()[:3], 0.125, _lib.FLASH_VARIANT[variant], *extra,
                                     _lib.stream_ptr(q.device)))
    return out


@pytest.mark.parametrize("variant", ["fh", "hh"])
@pytest.mark.parametrize("B,N,H", [(1, 6145, 16), (2, 2500, 11), (20, 300, 16), (1, 257, 6)])
def test_static_workspace_matches_the_caller_workspace_entry_point(oracle, B, N, H, variant):
    from fastbb_b200 import _lib
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(7 * B + N + H)
    qkv = torch.randn(B, N, 3, H, 64, generator=g).half().to(dev)
    q, k, v = qkv.unbind(2)
    need = _lib.load().fbb_flash64_workspace_bytes(B, N, H)          # 0 for the small shape: nothing is split there
    ws = torch.zeros(max(need, 16), dtype=torch.uint8, device=dev)
    want = _call("fbb_flash64_f16_ws", q, k, v, torch.empty(B, N, H, 64, dtype=torch.float16, device=dev), variant,
                 ws.data_ptr() if need else None, ws.numel() if need else 0)
    plain = _call("fbb_flash64_f16", q, k, v, torch.empty_like(want), variant)
    first = _call("fbb_flash64_f16_static", q, k, v, torch.empty_like(want), variant)
    second = _call("fbb_flash64_f16_static", q, k, v, torch.empty_like(want), variant)   # straight after, same array
    torch.cuda.synchronize()
    assert torch.equal(first, want)              # same schedule, same arithmetic: bit-identical
    assert torch.equal(second, want)
    assert (first.float() - plain.float()).norm() / plain.float().norm() < 3e-4
    if (B, N, H) == (2, 2500, 11):               # and against the CPU oracle, not only against the library's other entry points
        q_, k_, v_ = qkv.cpu().unbind(2)
        assert oracle.rel_l2(first.cpu().float(), oracle.attention(q_, k_, v_, scale=0.125)) < 1e-3
    assert _lib.device_status() == (0, 0, 0, 0)


def test_static_workspace_entry_point_allocates_nothing_and_orders_on_the_stream():
    """What the entry point is for: after the first call (which looks the array's address up), further calls leave the
    device's free memory and torch's allocator untouched; on a side stream the clearing of the flag words is ordered with
    the kernel on that stream and the result is the same."""
    dev = torch.device("cuda", 0)
    B, N, H = 1, 6145, 16
    qkv = torch.randn(B, N, 3, H, 64, generator=torch.Generator().manual_seed(3)).half().to(dev)
    q, k, v = qkv.unbind(2)
    out = torch.empty(B, N, H, 64, dtype=torch.float16, device=dev)
    want = _call("fbb_flash64_f16_static", q, k, v, torch.empty_like(out), "fh").clone()   # first call on this device
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(dev)
    alloc0, reserved0 = torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
    for _ in range(5):
        _call("fbb_flash64_f16_static", q, k, v, out, "fh")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(dev)[0] == free0
    assert (torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)) == (alloc0, reserved0)
    assert torch.equal(out, want)
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    out2 = torch.empty_like(out)
    with torch.cuda.stream(side):
        for _ in range(3):
            _call("fbb_flash64_f16_static", q, k, v, out2, "fh")     # _call passes torch's current stream: the side stream
    side.synchronize()
    assert torch.equal(out2, want)


def test_static_workspace_entry_point_validates_like_the_others():
    """Arguments are checked before anything is enqueued or looked up: a rejected call leaves no trace on the stream."""
    from fastbb_b200 import _lib
    dev = torch.device("cuda", 0)
    q = torch.zeros(1, 8, 2, 64, dtype=torch.float16, device=dev)
    with pytest.raises(_lib.FastbbError):
        _lib.check(_lib.load().fbb_flash64_f16_static(None, q.data_ptr(), q.data_ptr(), q.data_ptr(), 1, 8, 2, *q.stride()[:3], *q.stride()[:3],
                                                      *q.stride()[:3], *q.stride()[:3], 0.125, 0, None))
    with pytest.raises(_lib.FastbbError):
        _lib.check(_lib.load().fbb_flash64_f16_static(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), 1, 8, 2, *q.stride()[:3],
                                                      *q.stride()[:3], *q.stride()[:3], *q.stride()[:3], 0.125, 9, None))


def test_attention_only_library_gives_the_same_attention():
    """The attention-only build (libfastbb_flash64.so) holds the same kernel: same bits as the full library."""
    from fastbb_b200 import _lib, build
    flash = _lib.load(build.build(flash_only=True))
    dev = torch.device("cuda", 0)
    qkv = torch.randn(1, 1370, 3, 16, 64, generator=torch.Generator().manual_seed(9)).half().to(dev)
    q, k, v = qkv.unbind(2)
    want = _call("fbb_flash64_f16", q, k, v, torch.empty(1, 1370, 16, 64, dtype=torch.float16, device=dev), "fh")
    got = torch.empty_like(want)
    _lib.check(flash.fbb_flash64_f16(q.data_ptr(), k.data_ptr(), v.data_ptr(), got.data_ptr(), 1, 1370, 16, *q.stride()[:3], *k.stride()[:3],
                                     *v.stride()[:3], *got.stride()[:3], 0.125, _lib.FLASH_VARIANT["fh"], _lib.stream_ptr(dev)))
    torch.cuda.synchronize()
    assert torch.equal(got, want)
