"""Host-side logic of the symmetric workspace (views, ring slots, containment, guard words) on plain CPU memory.

The kernels behind ``all_reduce_`` / ``gemm_all_reduce`` need GPUs with peer access; everything around them is
ordinary tensor arithmetic and is exercised here on a workspace whose storage is a CPU tensor.
"""
import pytest
import torch

from picotron_b200.comm import workspace as W


def _cpu_workspace(data_bytes: int) -> W.SymmetricWorkspace:
    ws = W.SymmetricWorkspace.__new__(W.SymmetricWorkspace)          # no symmetric-memory rendezvous
    ws.group, ws.world, ws.rank, ws.num_blocks = None, 2, 0, 4
    ws.data_bytes = data_bytes
    ws.staging_bytes, ws.staging_off, ws._body_bytes = 0, data_bytes, data_bytes      # no push staging area behind the data
    ws.storage = torch.zeros(W.FLAG_REGION + data_bytes + W.CANARY_BYTES, dtype=torch.uint8)
    ws.storage[W.FLAG_REGION - W.CANARY_BYTES:W.FLAG_REGION].fill_(W.CANARY_VALUE)
    ws.storage[W.FLAG_REGION + data_bytes:].fill_(W.CANARY_VALUE)
    ws.data = ws.storage[W.FLAG_REGION:W.FLAG_REGION + data_bytes]
    ws.epoch, ws._gemm_clusters = 0, None
    ws._ring_slot_bytes = ws._ring_slots = ws._ring_next = 0
    return ws


def test_views_and_ring_slots_stay_inside_the_data_region():
    ws = _cpu_workspace(1 << 16)
    v = ws.view(4096, (8, 16), torch.float32)
    assert v.shape == (8, 16) and v.data_ptr() == ws.data.data_ptr() + 4096
    with pytest.raises(AssertionError):
        ws.view(8, (4,), torch.float32)                               # offsets are 16-byte aligned
    with pytest.raises(AssertionError):
        ws.view(0, (1 << 16,), torch.float32)                         # 256 KiB do not fit 64 KiB
    assert ws.ring_alloc((4, 4), torch.bfloat16) is None              # no ring configured yet
    ws.configure_ring(4, 8192)
    ptrs = [ws.ring_alloc((32, 64), torch.bfloat16).data_ptr() - ws.data.data_ptr() for _ in range(6)]
    assert ptrs == [0, 8192, 16384, 24576, 0, 8192]                   # round robin over the four slots
    assert ws.ring_alloc((64, 128), torch.bfloat16) is None           # 16 KiB does not fit an 8 KiB slot
    with pytest.raises(AssertionError):
        ws.configure_ring(16, 8192)                                   # 128 KiB of slots in a 64 KiB region


def test_guard_words_detect_writes_behind_either_region():
    ws = _cpu_workspace(4096)
    ws.check_canaries()
    ws.data.fill_(7)                                                  # writing the whole data region is fine
    ws.storage[:W.FLAG_REGION - W.CANARY_BYTES].fill_(9)              # and so are all flag words
    ws.check_canaries()
    ws.storage[W.FLAG_REGION + 4096 + 3] = 0                          # one byte behind the data region
    with pytest.raises(RuntimeError, match="data region"):
        ws.check_canaries()
    ws.storage[W.FLAG_REGION + 4096 + 3] = W.CANARY_VALUE
    ws.storage[W.FLAG_REGION - 1] = 1                                 # last byte of the flag region's guard
    with pytest.raises(RuntimeError, match="flag region"):
        ws.check_canaries()


def test_scratch_area_alternates_between_two_halves_inside_the_data_region():
    ws = _cpu_workspace(1 << 16)
    ws.configure_scratch(32768, 16384)
    assert ws.can_exchange_ce_stats(512) and not ws.can_exchange_ce_stats(1024)      # 3 fp32 vectors per half of 8 KiB
    with pytest.raises(AssertionError):
        ws.configure_scratch(61440, 8192)                                           # would run past the data region


def test_flag_region_layout_leaves_room_for_the_guard_words():
    # 16 KiB of barrier flags + per-tile flags of the fused GEMM+all-reduce (1024 tiles x 2 halves x (8 + 1) words)
    used = 16384 + 1024 * 2 * 9 * 4
    assert W.FLAG_BYTES + 8 <= 16384                      # barrier flags, then the two control words (call counter, arrivals)
    assert W.CTRL_OFFSET == W.FLAG_BYTES
    assert used <= W.FLAG_REGION - W.CANARY_BYTES


def _node_check_worker(rank, world, fake_hosts):
    import socket
    from picotron_b200.comm import workspace as W
    import torch.distributed as dist
    if fake_hosts:
        socket.gethostname = lambda: f"node{rank // 2}"            # ranks 0,1 on one host, 2,3 on another
    whole = W.group_is_on_one_node(dist.group.WORLD)
    pair = dist.new_group([0, 1])
    other = dist.new_group([2, 3])
    mine = pair if rank < 2 else other
    created = W.try_create(dist.group.WORLD, 1024) if fake_hosts else "not tried"
    return {"whole": whole, "pair": W.group_is_on_one_node(mine), "created": created if created is None else "object"}


def test_groups_that_span_hosts_do_not_get_a_peer_memory_workspace():
    from dist_utils import run_distributed
    for r in run_distributed(_node_check_worker, 4, False):
        assert r["whole"] and r["pair"]
    for r in run_distributed(_node_check_worker, 4, True):
        assert not r["whole"] and r["pair"] and r["created"] is None   # refused before any symmetric-memory call
