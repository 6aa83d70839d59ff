"""Placement planner against the cases the reference's own planner tests hold
(src/format/load_plan.rs:714-1130), on index fixtures with the same tensors
(src/format/ggufrs.rs:3203-3348: a 128-byte F32 shared tensor plus Q8_0 layer tensors)."""
import pytest


def _pair_index(lp):
    # llm of test_gguf_pair: token_embd F32 [32] (128 B), blk.0 / blk.1 Q8_0 [32] (34 B each)
    return lp.PackageIndex.from_tensor_table(
        [("token_embd.weight", [32], 0), ("blk.0.weight", [32], 8), ("blk.1.weight", [32], 8)], block_count=2)


def _row_index(lp, rows, row_elements):
    # test_q8_row_package: token_embd F32 [32], blk.0.weight Q8_0 [row_elements, rows]
    return lp.PackageIndex.from_tensor_table(
        [("token_embd.weight", [32], 0), ("blk.0.weight", [row_elements, rows], 8)], block_count=1)


def test_index_follows_the_exporter_layout(rmi):
    lp = rmi.load_plan
    idx = lp.PackageIndex.from_tensor_table(
        [("output_norm.weight", [32], 0), ("blk.1.b", [32], 8), ("blk.0.z", [32], 8), ("blk.0.a", [32, 3], 8),
         ("token_embd.weight", [32], 0)], block_count=2)
    assert [(s.kind, s.layer) for s in idx.segments] == [(lp.SHARED, None), (lp.LAYER, 0), (lp.LAYER, 1)]
    assert [(t.name, t.segment_id, t.segment_offset, t.byte_len) for t in idx.tensors] == [
        ("output_norm.weight", 0, 0, 128), ("token_embd.weight", 0, 128, 128),
        ("blk.0.a", 1, 0, 102), ("blk.0.z", 1, 128, 34), ("blk.1.b", 2, 0, 34)]
    assert lp.layer_index("blk.12.attn_q.weight") == 12
    assert lp.layer_index("blk.3.") is None and lp.layer_index("blk.x.w") is None and lp.layer_index("token") is None
    with pytest.raises(lp.PlanError):
        lp.PackageIndex.from_tensor_table([("blk.2.w", [32], 8), ("t", [32], 0)], block_count=2)


def test_layer_split_keeps_layers_whole_and_shared_on_primary(rmi):
    lp = rmi.load_plan
    idx = _pair_index(lp)
    devices = [lp.LogicalDevice("cpu0", 128 + 34), lp.LogicalDevice("cpu1", 34)]
    plan = lp.build_load_plan(idx, [0], devices, "cpu0", lp.LAYER_SPLIT)
    assert plan == lp.build_load_plan(idx, [0], devices, "cpu0", lp.LAYER_SPLIT)
    assert all(p.slice is lp.WHOLE for p in plan.placements)
    by_name = {p.tensor_name: p.device_id for p in plan.placements}
    assert by_name == {"token_embd.weight": "cpu0", "blk.0.weight": "cpu0", "blk.1.weight": "cpu1"}
    assert plan.used_bytes("cpu0") == 162 and plan.used_bytes("cpu1") == 34


def test_tensor_split_uses_only_complete_quantized_rows(rmi):
    lp = rmi.load_plan
    idx = _row_index(lp, 4, 32)
    devices = [lp.LogicalDevice("cpu0", 196), lp.LogicalDevice("cpu1", 68)]
    plan = lp.build_load_plan(idx, [0], devices, "cpu0", lp.TENSOR_SPLIT)
    plan.validate(idx)
    rows = [p for p in plan.placements if p.tensor_name == "blk.0.weight"]
    assert [p.slice for p in rows] == [(0, 2), (2, 4)]
    assert [p.device_id for p in rows] == ["cpu0", "cpu1"]
    assert all((p.segment_byte_range[1] - p.segment_byte_range[0]) % 34 == 0 for p in rows)
    assert plan.rows_on("blk.0.weight", "cpu1") == [(2, 4)]


def test_row_layout_rejects_incomplete_quantization_blocks(rmi):
    lp = rmi.load_plan
    with pytest.raises(lp.UnsplittableTensor):
        lp.row_layout(lp.TensorRecord(0, 0, "bad", (31, 2), 8, 0, 68))
    assert lp.row_layout(lp.TensorRecord(0, 0, "ok", (64, 3), 8, 0, 204)) == (3, 68)
    assert lp.row_layout(lp.TensorRecord(0, 0, "k", (256, 2), 12, 0, 288)) == (2, 144)
    assert lp.row_layout(lp.TensorRecord(0, 0, "k6", (256, 2), 14, 0, 420)) == (2, 210)
    with pytest.raises(lp.PlanError):
        lp.row_layout(lp.TensorRecord(0, 0, "len", (32, 2), 8, 0, 67))


def test_tensor_split_keeps_rank_one_layer_tensors_whole(rmi):
    lp = rmi.load_plan
    idx = _pair_index(lp)
    devices = [lp.LogicalDevice("cpu0", 128), lp.LogicalDevice("cpu1", 68)]
    plan = lp.build_load_plan(idx, [0], devices, "cpu0", lp.TENSOR_SPLIT)
    layers = [p for p in plan.placements if p.tensor_name.startswith("blk.")]
    assert len(layers) == 2
    assert all(p.device_id == "cpu1" and p.slice is lp.WHOLE for p in layers)


def test_planning_reports_capacity_and_row_failures(rmi):
    lp = rmi.load_plan
    with pytest.raises(lp.CapacityExceeded):
        lp.build_load_plan(_pair_index(lp), [0], [lp.LogicalDevice("cpu0", 127)], "cpu0", lp.LAYER_SPLIT)
    with pytest.raises(lp.CapacityExceeded):
        lp.build_load_plan(_pair_index(lp), [0], [lp.LogicalDevice("cpu0", 128 + 34)], "cpu0", lp.LAYER_SPLIT)
    devices = [lp.LogicalDevice("cpu0", 128), lp.LogicalDevice("cpu1", 34)]
    with pytest.raises(lp.UnsplittableTensor) as e:
        lp.build_load_plan(_row_index(lp, 2, 64), [0], devices, "cpu0", lp.TENSOR_SPLIT)
    assert e.value.row_bytes == 68


def test_planning_rejects_ambiguous_devices_and_components(rmi):
    lp = rmi.load_plan
    idx = _pair_index(lp)
    one = [lp.LogicalDevice("cpu", 1024)]
    for args in (([0], [lp.LogicalDevice("cpu", 1024)] * 2, "cpu"), ([0], one, "missing"), ([0, 0], one, "cpu"),
                 ([2 ** 32 - 1], one, "cpu"), ([0], [], "cpu"), ([0], [lp.LogicalDevice("", 1)], "")):
        with pytest.raises(lp.PlanError):
            lp.build_load_plan(idx, args[0], args[1], args[2], lp.LAYER_SPLIT)


def test_validation_rejects_missing_overlapping_or_misaligned_rows(rmi):
    lp = rmi.load_plan
    idx = _row_index(lp, 4, 32)
    devices = [lp.LogicalDevice("cpu0", 196), lp.LogicalDevice("cpu1", 68)]
    plan = lp.build_load_plan(idx, [0], devices, "cpu0", lp.TENSOR_SPLIT)
    from dataclasses import replace
    with pytest.raises(lp.PlanError):
        lp.with_placements(plan, plan.placements[:-1]).validate(idx)
    overlap = [replace(p, slice=(1, 4)) if p.slice == (2, 4) else p for p in plan.placements]
    with pytest.raises(lp.PlanError):
        lp.with_placements(plan, overlap).validate(idx)
    cut = [replace(p, segment_byte_range=(p.segment_byte_range[0], p.segment_byte_range[1] - 1))
           if p.slice == (0, 2) else p for p in plan.placements]
    with pytest.raises(lp.PlanError):
        lp.with_placements(plan, cut).validate(idx)


def test_validation_rejects_forged_device_capacity_and_layer_rules(rmi):
    lp = rmi.load_plan
    from dataclasses import replace
    idx = _pair_index(lp)
    devices = [lp.LogicalDevice("cpu0", 162), lp.LogicalDevice("cpu1", 34)]
    plan = lp.build_load_plan(idx, [0], devices, "cpu0", lp.LAYER_SPLIT)
    forged = [replace(p, device_id="cpu1") if p.tensor_name == "token_embd.weight" else p for p in plan.placements]
    with pytest.raises(lp.PlanError):                       # shared tensor off the primary device
        lp.with_placements(plan, forged).validate(idx)
    unknown = [replace(p, device_id="gpu9") if p.tensor_name == "blk.1.weight" else p for p in plan.placements]
    with pytest.raises(lp.PlanError):
        lp.with_placements(plan, unknown).validate(idx)
    crowd = [replace(p, device_id="cpu1") if p.tensor_name == "blk.0.weight" else p for p in plan.placements]
    with pytest.raises(lp.CapacityExceeded):                # both layers on the 34-byte device
        lp.with_placements(plan, crowd).validate(idx)
    back = [replace(p, device_id={"blk.0.weight": "cpu1", "blk.1.weight": "cpu0"}.get(p.tensor_name, p.device_id))
            for p in plan.placements]
    roomy = replace(plan, devices=[lp.LogicalDevice("cpu0", 1024), lp.LogicalDevice("cpu1", 1024)])
    with pytest.raises(lp.PlanError):                       # device order goes backwards
        lp.with_placements(roomy, back).validate(idx)
    rows = [replace(p, slice=(0, 1)) if p.tensor_name == "blk.0.weight" else p for p in plan.placements]
    with pytest.raises(lp.PlanError):                       # LayerSplit placements must be whole
        lp.with_placements(plan, rows).validate(idx)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_balanced_devices_cut_one_matrix_into_equal_row_ranges(rmi, world):
    lp = rmi.load_plan
    n, k = 32768, 8192                                      # the column-sharded matmul's weight
    idx = lp.PackageIndex.from_tensor_table([("token_embd.weight", [32], 0), ("blk.0.weight", [k, n], 8)], 1)
    devices = lp.balanced_devices(idx, world)
    plan = lp.build_load_plan(idx, [0], devices, devices[0].id, lp.TENSOR_SPLIT)
    for r in range(world):
        got = plan.rows_on("blk.0.weight", f"cuda{r}")
        want = rmi.sharding.shard_rows(n, world, r)
        assert got == [lp.WHOLE if world == 1 else want]


def test_plan_from_a_gguf_file_covers_every_tensor(rmi, tmp_path):
    lp = rmi.load_plan
    import numpy as np
    g = rmi.gguf
    path = str(tmp_path / "m.gguf")
    w0 = rmi.synth.q8_0_weight_rows(24, 64, seed=1, row_begin=0, row_end=24)
    w1 = rmi.synth.q8_0_weight_rows(8, 64, seed=2, row_begin=0, row_end=8)
    g.write_gguf(path, [("general.architecture", g.T_STR, "qwen3"), ("qwen3.block_count", g.T_U32, 2)],
                 [("token_embd.weight", [32], g.GGML_F32, np.zeros(128, np.uint8)),
                  ("blk.0.ffn_up.weight", [64, 24], g.GGML_Q8_0, w0),
                  ("blk.0.ffn_norm.weight", [64], g.GGML_F32, np.zeros(256, np.uint8)),
                  ("blk.1.ffn_up.weight", [64, 8], g.GGML_Q8_0, w1)])
    idx = lp.PackageIndex.from_gguf_file(path)
    devices = lp.balanced_devices(idx, 3, slack_rows=1)
    plan = lp.build_load_plan(idx, [0], devices, "cuda0", lp.TENSOR_SPLIT)
    plan.validate(idx)
    total = sum(plan.used_bytes(d.id) for d in devices)
    assert total == sum(t.byte_len for t in idx.tensors)
    assert len({p.device_id for p in plan.placements}) == 3
