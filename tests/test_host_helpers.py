"""Host-side decisions that need no GPU: scratch buffers and their views, the rule that cuts decode attention's keys
over CTAs, the decode batch buckets, and the cache's serial numbers (what decode graphs are kept by)."""
import pytest
import torch

from xpu_serve_b200.cache import Cache
from xpu_serve_b200.engine.model import _bucket, _kv_bucket
from xpu_serve_b200.engine.runtime import Workspace
from xpu_serve_b200.parts.attention import decode_splits
from xpu_serve_b200.parts.base import KVNeed, StateNeed


def test_workspace_hands_out_the_same_view_until_the_buffer_grows():
    ws = Workspace(torch.device("cpu"))
    a = ws.get("x", (3, 4), torch.float32)
    assert a.shape == (3, 4) and ws.get("x", [3, 4], torch.float32) is a          # the same view again, list or tuple
    b = ws.get("x", (2, 4), torch.float32)
    assert b.data_ptr() == a.data_ptr() and b.shape == (2, 4)                      # one buffer per name and type
    assert ws.get("x", (3, 4), torch.bfloat16).data_ptr() != a.data_ptr()          # another type, another buffer
    a.fill_(7.0)
    big = ws.get("x", (10, 4), torch.float32)                                      # grows: a new buffer
    assert big.data_ptr() != a.data_ptr()
    again = ws.get("x", (3, 4), torch.float32)
    assert again is not a and again.data_ptr() == big.data_ptr(), "a view of the old buffer was handed out again"
    assert ws.get("empty", (0, 5), torch.float32).shape == (0, 5)
    ws.frozen = True
    assert ws.get("x", (10, 4), torch.float32) is big                              # fits: fine when frozen
    with pytest.raises(RuntimeError, match="frozen"):
        ws.get("x", (11, 4), torch.float32)
    with pytest.raises(RuntimeError, match="frozen"):
        ws.get("never seen", (1,), torch.float32)


def test_decode_splits_rule():
    slots = 444                                        # 148 SMs x 3 CTAs
    for tiles in (1, 8, 64, 128, 512, 4096):
        for blocks in (1, 2, 33, 64, 384, 2048):
            n = decode_splits(tiles, blocks, slots)
            assert 1 <= n <= min(blocks, 64), (tiles, blocks, n)
    assert decode_splits(8, 1, slots) == 1                                         # nothing to cut
    assert decode_splits(4096, 33, slots) == 1                                     # the tiles alone are many rounds
    assert decode_splits(64, 33, slots) == 6                                       # 8 sequences x 8 kv heads: one round of 384
    assert 8 <= decode_splits(8, 33, slots) <= 16                                  # one sequence: the combine's cost caps it
    assert decode_splits(8, 2048, slots) > 32                                      # one long sequence: fill the device
    assert decode_splits(8, 2048, slots) * 8 <= slots                              # ... in one round
    # more CTA slots never ask for fewer parts of a long sequence
    assert decode_splits(8, 2048, 2 * slots) >= decode_splits(8, 2048, slots)


def test_decode_batch_buckets():
    assert [_bucket(n) for n in (1, 5, 8, 9, 16, 17, 63, 64, 65, 96, 97)] == [1, 5, 8, 16, 16, 24, 64, 64, 96, 96, 128]
    assert all(_bucket(n) >= n for n in range(1, 300))


def test_key_length_bounds_of_decode_graphs():
    assert [_kv_bucket(n, 1 << 20) for n in (1, 1024, 1025, 1536, 1537, 2048, 2049, 3073, 100000)] == \
        [1024, 1024, 1536, 1536, 2048, 2048, 3072, 4096, 131072]
    assert all(n <= _kv_bucket(n, 1 << 20) < 2 * max(n, 1024) for n in range(1, 5000, 7))
    assert _kv_bucket(5, 300) == 300 and _kv_bucket(3100, 3500) == 3500       # never beyond the cache's limit


def test_every_cache_has_a_serial_number_of_its_own():
    def make():
        return Cache([StateNeed((2, 8)), KVNeed(2, 16, 0)], [None, None], 256, dtype=torch.float32, device="cpu")
    seen = set()
    for _ in range(5):
        c = make()
        assert c.serial not in seen
        seen.add(c.serial)
        del c                                          # the next one may get the same id(), never the same serial
