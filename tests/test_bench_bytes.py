"""The algorithmic byte counts behind the reported roofline fractions, against constants worked
out by hand from the formats: W4A16 g128 stores K N / 2 bytes of codes, a bf16 scale and half a
byte of zero point per group of 128 weights; an INT8 KV token costs 2 x 8 x 128 code bytes and
2 x 8 f32 scales per layer."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import bench  # noqa: E402
import microbench  # noqa: E402


def test_weight_side_bytes_of_the_microbenchmark_shapes():
    assert bench.w4_bytes(4096, 4096) == 8_716_288
    assert bench.w4_bytes(14336, 4096) == bench.w4_bytes(4096, 14336) == 30_507_008
    assert bench.w4_bytes(128256, 4096) == 4096 * 128256 // 2 + 32 * 128256 * 2 + 32 * 128256 // 2
    for n, k in [(4096, 4096), (14336, 4096), (4096, 14336), (128256, 4096)]:
        assert microbench.w4_bytes(n, k) == bench.w4_bytes(n, k)


def test_bytes_of_one_large_decode_step():
    assert bench.step_weight_bytes(bench.LARGE) == 3_694_071_808
    assert bench.kv_bytes_per_token(bench.LARGE) == 32 * 2112
    shapes = bench.linear_shapes(bench.LARGE)
    assert shapes["wq"] == (4096, 4096) and shapes["wk"] == shapes["wv"] == (1024, 4096)
    assert shapes["w_gate"] == shapes["w_up"] == (14336, 4096) and shapes["w_down"] == (4096, 14336)
