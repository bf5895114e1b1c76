"""Host core (C++): distributed-states algebra, comm classification, reshard planner, schedules, symbols."""
import itertools

import numpy as np
import pytest

from hotspa_ae_b200 import core as C

DS = C.DistributedStates
K = C._C


def test_ds_states_order_and_index_maps():
    ds = DS(8, {0: 2, 1: 2, -1: 2}, [-1, 0, 1])             # weights: dup slow, splits fast
    assert ds.device_num == 8 and ds.get_dim(0) == 2 and ds.get_dim(1) == 2 and ds.get_dim(-1) == 2
    assert ds.get_dim(-2) == 1 and not ds.is_pure_duplicate
    # digits are peeled from the last order entry: device 5 = (dup 1, dim0 0, dim1 1)
    assert dict(ds.map_device_to_state_index(5)) == {-1: 1, 0: 0, 1: 1}
    # duplicate-group index counts only the non-negative dims
    assert [ds.get_dup_group_index(i) for i in range(8)] == [0, 1, 2, 3, 0, 1, 2, 3]
    # devices that differ only in the dup digit
    assert list(ds.get_devices_by_dim(-1, 1, list(range(8)))) == [1, 5]
    assert list(ds.get_devices_by_dim(1, 6, list(range(8)))) == [6, 7]
    with pytest.raises(Exception):
        DS(8, {0: 3}, [0])                                    # product must equal device_num
    assert DS(4, {-1: 4}, [-1]).is_pure_duplicate


@pytest.mark.parametrize("shape,states,order", [([16, 12], {0: 2, 1: 2, -1: 2}, [-1, 0, 1]),
                                                ([24, 8], {0: 4, -1: 2}, [0, -1]),
                                                ([8, 8], {1: 8}, [1])])
def test_local_slices_tile_the_tensor_once_per_replica(shape, states, order):
    n = int(np.prod(list(states.values())))
    ds = DS(n, states, order)
    cover = np.zeros(shape, dtype=np.int32)
    for dev in range(n):
        sl = ds.local_slice(shape, dev)
        assert [s for _, s in sl] == list(ds.local_shape(shape))
        cover[tuple(slice(o, o + s) for o, s in sl)] += 1
    assert (cover == states.get(-1, 1)).all()


def test_collective_pattern_checks_and_classification():
    ranks = [0, 1, 2, 3]
    partial = DS(4, {-2: 2, 0: 2}, [0, -2])
    dup = DS(4, {-1: 2, 0: 2}, [0, -1])
    split0 = DS(4, {0: 4}, [0])
    assert partial.check_allreduce(dup) and partial.check_reducescatter(split0) and split0.check_allgather(dup)
    U = C.DistributedStatesUnion
    name = lambda a, b, g2=ranks: C.comm_type_name(C.classify_comm(U([a]), ranks, U([b]), g2, 0))  # noqa: E731
    assert name(partial, dup) == C.comm_type_name(K.COMM_ALL_REDUCE)
    assert name(partial, split0) == C.comm_type_name(K.COMM_REDUCE_SCATTER)
    assert name(split0, dup) == C.comm_type_name(K.COMM_ALL_GATHER)
    assert name(dup, dup) == C.comm_type_name(K.COMM_UNUSED)
    assert name(dup, dup, [4, 5, 6, 7]) == C.comm_type_name(K.COMM_P2P)
    assert name(split0, dup, [4, 5, 6, 7]) == C.comm_type_name(K.COMM_BATCHED_SEND_RECV)


def test_linear_ds_deduction_column_and_row_parallel():
    x_dup = DS(4, {0: 2, -1: 2}, [0, -1])                     # activations: dp 2, replicated over tp 2
    w_col = DS(4, {-1: 2, 0: 2}, [-1, 0])                     # W [out, in] split on out
    y = C.deduce_linear(x_dup, w_col, False, True)
    assert y.get_dim(0) == 2 and y.get_dim(1) == 2 and y.get_dim(-2) == 1
    x_split = DS(4, {0: 2, 1: 2}, [0, 1])                     # activations split on features
    w_row = DS(4, {-1: 2, 0: 2}, [-1, 0])                     # W [in, out] split on in
    y2 = C.deduce_linear(x_split, w_row, False, False)
    assert y2.get_dim(-2) == 2 and y2.get_dim(0) == 2         # partial over tp


def _layouts(shape, dp, tp, pp, world):
    """Column-parallel weight of stage 0 under (dp, tp, pp): ranks of the first stage, dup dp x split0 tp."""
    width = world // pp
    ds = DS(width, {-1: dp, 0: tp}, [-1, 0]) if dp * tp > 1 else DS(1, {-1: 1}, [-1])
    return ds, list(range(width))


@pytest.mark.parametrize("src,dst", list(itertools.permutations([(8, 1, 1), (2, 2, 2), (1, 4, 2), (4, 2, 1)], 2)))
def test_reshard_plan_properties(src, dst):
    shape, world = [64, 32], 8
    s_ds, s_ranks = _layouts(shape, *src, world)
    d_ds, d_ranks = _layouts(shape, *dst, world)
    s_regs = C.regions_of(shape, s_ds, s_ranks, -1)
    d_regs = C.regions_of(shape, d_ds, d_ranks, -1)
    pl = C.ReshardPlanner(world, K.SENDER_BALANCED)
    pl.add_tensor_regions(0, s_regs, d_regs, False)
    # execute the plan on numpy shards: every destination shard must come out complete
    full = np.arange(shape[0] * shape[1], dtype=np.float32).reshape(shape)
    src_sh = {r: full[r0:r1, c0:c1].copy() for r, r0, r1, c0, c1 in s_regs}
    dst_sh = {r: np.full((r1 - r0, c1 - c0), -1, np.float32) for r, r0, r1, c0, c1 in d_regs}
    sent = recv = 0
    for c in pl.copies():
        s = src_sh[c.src_rank].reshape(-1)
        d = dst_sh[c.dst_rank].reshape(-1)
        for row in range(c.rows):
            d[c.dst_off + row * c.dst_ld:c.dst_off + row * c.dst_ld + c.row_elems] = \
                s[c.src_off + row * c.src_ld:c.src_off + row * c.src_ld + c.row_elems]
        if c.src_rank != c.dst_rank:
            sent += c.rows * c.row_elems
            recv += c.rows * c.row_elems
    for r, r0, r1, c0, c1 in d_regs:
        np.testing.assert_array_equal(dst_sh[r], full[r0:r1, c0:c1])
    st = pl.stats
    assert sum(st.sent_elems) == sum(st.recv_elems) == sent == st.remote_elems
    # a rank never fetches remotely what it already holds
    if src == dst:
        assert st.remote_elems == 0


def test_gradient_plan_gathers_every_replica():
    shape, world = [32, 16], 4
    s_ds = DS(4, {-1: 4}, [-1])                               # dp4: four replicas hold partial sums of the whole tensor
    d_ds = DS(4, {0: 4}, [0])                                 # home: split in four
    s_regs = C.regions_of(shape, s_ds, [0, 1, 2, 3], -1)
    d_regs = C.regions_of(shape, d_ds, [0, 1, 2, 3], 0)
    pl = C.ReshardPlanner(world, K.SENDER_BALANCED)
    pl.add_tensor_regions(0, s_regs, d_regs, True)
    per_dst = {}
    for c in pl.copies():
        per_dst.setdefault(c.dst_rank, set()).add(c.src_rank)
    assert all(v == {0, 1, 2, 3} for v in per_dst.values()) and len(per_dst) == 4


def test_pipeline_schedules():
    for stages, nmb in [(2, 4), (4, 8), (4, 2), (1, 3)]:
        for s in range(stages):
            t = C.schedule_1f1b(stages, s, nmb)
            fw = [m for f, m in t if f]
            bw = [m for f, m in t if not f]
            assert fw == list(range(nmb)) and bw == list(range(nmb))
            # a backward never precedes its forward, and at most (stages - s) micro-batches are in flight
            live = peak = 0
            for f, m in t:
                live += 1 if f else -1
                peak = max(peak, live)
                assert live >= 0
            assert peak <= min(nmb, stages - s)
            g = C.schedule_gpipe(stages, s, nmb)
            assert [m for f, m in g if f] == list(range(nmb)) and all(f for f, _ in g[:nmb])


def test_symbols_packer_and_arena():
    a, b = C.IntSymbol(6), C.IntSymbol(4)
    c = a * b + a / C.IntSymbol(2) - b % C.IntSymbol(3)
    assert c.data == 24 + 3 - 1
    a.set_data(10)
    assert c.data == 40 + 5 - 1                               # lazy: follows its leaves
    buckets = C.bucket_and_pack([5, 9, 2, 7, 3, 12], [12, 6, 0], 0, False)
    assert sorted(i for bk in buckets for i in bk.members) == list(range(6))
    assert all(sum([5, 9, 2, 7, 3, 12][i] for i in row) <= bk.max_len for bk in buckets for row in bk.rows)
    assign = C.balance_rows([10, 9, 8, 1, 1, 1], 2)
    loads = [sum([10, 9, 8, 1, 1, 1][i] for i in a) for a in assign]
    assert abs(loads[0] - loads[1]) <= 4 and sum(loads) == 30          # longest-processing-time-first
    offs, total = C.plan_arena([10, 300, 5], 256)
    assert offs == [0, 256, 768] and total == 1024


def test_hetero_strategy_config_and_unions():
    import hetu as ht
    from hotspa_ae_b200.parallel.strategy_config import find_config, generate_llama_hetero_3d_config
    pipes = [[{"ranks": [0, 1, 2, 3], "layers": 4}], [{"ranks": [4, 5], "layers": 2}, {"ranks": [6, 7], "layers": 2}]]
    cfg = generate_llama_hetero_3d_config(4, pipes, zero=False)
    assert cfg["devices"] == list(range(8)) and len(cfg["llama"]["blocks"]) == 4
    qkv0 = find_config(cfg, "qkv", 0)
    qkv3 = find_config(cfg, "qkv", 3)
    assert qkv0["device_group_union"] == [[0, 1, 2, 3], [4, 5]] and qkv3["device_group_union"] == [[0, 1, 2, 3], [6, 7]]
    assert qkv0["split"] == {"1": [4, 2]} and qkv0["dup"] == [2, 2]
    qkv0["zero"] = False
    u, groups = ht.nn.config2ds(qkv0)
    assert u.hetero_dim == -1 and [g.ranks() for g in groups] == [[0, 1, 2, 3], [4, 5]]
    a, b = u.get_local(0), u.get_local(1)
    assert (a.device_num, a.get_dim(1), a.get_dim(-1)) == (4, 4, 1) and (b.device_num, b.get_dim(1)) == (2, 2)
    # gradient sync of this parameter: rank 4 holds columns [0, 1/2) = micro-blocks 0 and 1 of the 4-way split
    plan = C.split_comm_groups([a, b], [[0, 1, 2, 3], [4, 5]], 4)
    assert plan.split_dim == 1 and plan.micro_blocks == 2 and plan.groups == [[[0, 4]], [[1, 4]]]
    plan = C.split_comm_groups([a, b], [[0, 1, 2, 3], [4, 5]], 3)
    assert plan.micro_blocks == 1 and plan.groups == [[[3, 5]]]
    u_in, _ = ht.nn.config2ds(cfg["input"])
    assert u_in.hetero_dim == 0 and u_in.get_local(1).get_dim(0) == 1 and u_in.get(1).get_dim(0) == 2
    with pytest.raises(ValueError):
        generate_llama_hetero_3d_config(4, [[{"ranks": [0], "layers": 4}], [{"ranks": [0], "layers": 4}]])


def _descriptors_oracle(rows, unit_bytes, rank, world):
    """Plain-Python statement of the descriptor rules (what the C++ builder must reproduce exactly)."""
    by_src = {}
    for s_ptr, d_ptr, r, rb, sld, dld, src_rank in rows:
        if sld == rb and dld == rb:
            r, rb, sld, dld = 1, rb * r, rb * r, rb * r
        bucket = by_src.setdefault(src_rank, [])
        if r == 1 and rb > unit_bytes:
            for k in range((rb + unit_bytes - 1) // unit_bytes):
                b0 = k * unit_bytes
                bucket.append((s_ptr + b0, d_ptr + b0, 1, min(unit_bytes, rb - b0), 0, 0, 1))
        else:
            ur = max(1, unit_bytes // max(rb, 1))
            for k in range((r + ur - 1) // ur):
                r0 = k * ur
                bucket.append((s_ptr + r0 * sld, d_ptr + r0 * dld, min(ur, r - r0), rb, sld, dld, ur))
    order = sorted(by_src, key=lambda q: (q - rank - 1) % world)
    cursors, descs = {q: 0 for q in order}, []
    left = sum(len(v) for v in by_src.values())
    while left:
        for q in order:
            if cursors[q] < len(by_src[q]):
                descs.append(by_src[q][cursors[q]])
                cursors[q] += 1
                left -= 1
    arr = np.array([d[:6] for d in descs], dtype=np.int64).reshape(-1, 6)
    ur = np.array([d[6] for d in descs], dtype=np.int32)
    prefix = np.concatenate([[0], np.cumsum([(d[2] + d[6] - 1) // d[6] for d in descs])]).astype(np.int32)
    return arr, ur, prefix


@pytest.mark.parametrize("rank,world,seed", [(0, 8, 0), (5, 8, 1), (1, 2, 2), (3, 4, 3)])
def test_reshard_descriptor_builder_matches_the_rules(rank, world, seed):
    rng = np.random.default_rng(seed)
    rows = []
    for _ in range(200):
        src_rank = int(rng.integers(0, world))
        rb = int(rng.choice([64, 1024, 8192, 300000, 1 << 20]))
        r = int(rng.integers(1, 400))
        full = bool(rng.integers(0, 2))
        sld = rb if full else rb * int(rng.integers(1, 4))
        dld = rb if full else rb * int(rng.integers(1, 4))
        rows.append((int(rng.integers(1, 1 << 40)) * 16, int(rng.integers(1, 1 << 40)) * 16, r, rb, sld, dld, src_rank))
    want = _descriptors_oracle(rows, 256 * 1024, rank, world)
    got = C.build_reshard_descriptors(np.array(rows, dtype=np.int64), 256 * 1024, rank, world)
    for g, w in zip(got, want):
        assert g.dtype == w.dtype and np.array_equal(g, w)
    # every byte of every rectangle is covered exactly once
    total = sum(r * rb for _, _, r, rb, _, _, _ in rows)
    assert int((got[0][:, 2] * got[0][:, 3]).sum()) == total
    assert got[2][-1] == sum((d[2] + u - 1) // u for d, u in zip(got[0], got[1]))
    with pytest.raises(ValueError):
        C.build_reshard_descriptors(np.array([[16, 32, 0, 64, 64, 64, 0]], dtype=np.int64), 1024, 0, 2)
