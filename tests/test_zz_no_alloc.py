"""The decode-attention entry point for callers that may not allocate device
memory (its split scratch is a fixed array inside the library): it must return
what the allocating entry point returns, on back-to-back calls that share the
array, and refuse problems larger than the array.  Collected last on purpose."""
import math

import numpy as np
import pytest
import torch

from helpers import pkg

pytestmark = pytest.mark.gpu


def _cache(p, lens, h=32, kvh=8, hd=128, dtype="int8", seed=40):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    cache = p.KVCache(max(lens), kvh, hd, h, batch=len(lens), dtype=dtype)
    for b, n in enumerate(lens):
        k = torch.randn((1, n, kvh, hd), generator=gen, device="cuda")
        v = torch.randn((1, n, kvh, hd), generator=gen, device="cuda")
        cache.update(k, v, row0=b)
    return cache


@pytest.mark.parametrize("dtype,act,h,kvh,hd", [("int8", torch.bfloat16, 32, 8, 128), ("f32", torch.float32, 32, 8, 128),
                                                 ("bf16", torch.bfloat16, 6, 2, 64)])
def test_static_scratch_entry_point_matches_allocating_one(dtype, act, h, kvh, hd):
    p = pkg()
    lens = [3000, 700]
    cache = _cache(p, lens, h=h, kvh=kvh, hd=hd, dtype=dtype)
    gen = torch.Generator(device="cuda").manual_seed(41)
    scale = 1 / math.sqrt(hd)
    qs = [torch.randn((2, h, hd), generator=gen, device="cuda").to(act) for _ in range(2)]
    want = [p.dispatch.attention_decode(cache, q, scale) for q in qs]
    outs = [torch.empty_like(q) for q in qs]
    # the first call on a device looks the array's address up; the calls measured below come after it
    p.dispatch.attention_decode_static(cache, qs[0], scale, outs[0])
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    # two calls in a row on one stream: the second reuses the scratch the first left behind
    for q, o in zip(qs, outs):
        p.dispatch.attention_decode_static(cache, q, scale, o)
    torch.cuda.synchronize()
    # the property the entry point exists for: the driver handed out no device memory
    assert torch.cuda.mem_get_info()[0] >= free_before
    for w, o in zip(want, outs):
        assert torch.isfinite(o.float()).all()
        err = (o.float() - w.float()).abs().max().item() / w.float().abs().max().item()
        assert err < 1e-6, err
    assert p.device_status() == 0


def test_static_scratch_rejects_oversized_problems():
    p = pkg()
    # Partials are indexed by the absolute cache row: rows 78..79 of an 80-row cache
    # with 56 context splits need 80 * 32 * 56 * 130 = 18.6 M floats, more than the
    # 2 Mi floats of the fixed array; rows 0..1 need 2 * 32 * 56 * 130 = 466 k.
    lens = [5000, 5000] + [8] * 76 + [5000, 5000]
    cache = _cache(p, lens, seed=42)
    q = torch.randn((2, 32, 128), device="cuda").to(torch.bfloat16)
    with pytest.raises(p.Ab2Error) as e:
        p.dispatch.attention_decode_static(cache, q, 0.1, torch.empty_like(q), row0=78)
    assert e.value.status == -4 and "static scratch" in str(e.value)
    ok = p.dispatch.attention_decode_static(cache, q, 0.1, torch.empty_like(q), row0=0)
    want = p.dispatch.attention_decode(cache, q, 0.1, row0=0)
    assert torch.equal(ok, want)
