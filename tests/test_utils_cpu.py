"""Data pipeline, logging / MFU arithmetic, debug helpers and profiling command builders (CPU only)."""
import json
import os
import tempfile

import numpy as np
import pytest
import torch


def test_pack_token_lists_and_token_array_dataset_round_trip():
    from state_space_models_neuron_b200.utils.data import TokenArrayDataset, create_pretraining_dataset, pack_token_lists
    docs = [[1, 2, 3], [4, 5, 6, 7, 8], [9], [10, 11, 12]]
    packed = pack_token_lists(docs, 4)
    assert packed.tolist() == [[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]] and packed.dtype == np.int32
    with tempfile.TemporaryDirectory() as d:
        np.save(os.path.join(d, "tokens.npy"), packed)
        ds = TokenArrayDataset(d)
        assert len(ds) == 3 and ds[1]["input_ids"].tolist() == [5, 6, 7, 8] and ds[1]["labels"].dtype == torch.int64
        # two data-parallel ranks see disjoint samples in a fixed order
        seen = []
        for rank in range(2):
            loader, sampler = create_pretraining_dataset(d, 1, 2, rank, seed=0)
            seen.append([b["input_ids"][0].tolist() for b in loader])
        assert seen[0] == [[1, 2, 3, 4]] and seen[1] == [[5, 6, 7, 8]]        # drop_last drops the odd third sample


def test_synthetic_dataset_is_deterministic_per_index():
    from state_space_models_neuron_b200.utils.data import SyntheticDataset
    a, b = SyntheticDataset(1000, 16, seed=3), SyntheticDataset(1000, 16, seed=3)
    assert torch.equal(a[5]["input_ids"], b[5]["input_ids"]) and not torch.equal(a[5]["input_ids"], a[6]["input_ids"])
    assert int(a[5]["input_ids"].max()) < 1000 and torch.equal(a[5]["labels"], a[5]["input_ids"])


def test_weight_decay_groups_follow_the_reference_rule():
    from state_space_models_neuron_b200.models import Mamba2Config, Mamba2ForCausalLM
    from state_space_models_neuron_b200.parallel import state as ps
    from state_space_models_neuron_b200.utils.data import get_param_groups_by_weight_decay
    ps.initialize_model_parallel(1)
    m = Mamba2ForCausalLM(Mamba2Config(num_heads=4, head_dim=32, vocab_size=64, hidden_size=64, state_size=32,
                                       num_hidden_layers=1, n_groups=1))
    decay, no_decay = get_param_groups_by_weight_decay(m, 0.1)
    names = {id(p): n for n, p in m.named_parameters()}
    nd = {names[id(p)] for p in no_decay["params"]}
    assert decay["weight_decay"] == 0.1 and no_decay["weight_decay"] == 0.0
    assert any(n.endswith("mixer.A_log") for n in nd) and any(n.endswith("mixer.dt_bias") for n in nd)
    assert any(n.endswith("mixer.norm.weight") for n in nd) and any(n.endswith("conv1d.bias") for n in nd)
    assert all(not n.endswith("in_proj.weight") and not n.endswith("out_proj.weight") for n in nd)


def test_throughput_window_and_mfu_formula():
    from state_space_models_neuron_b200.utils import logging as lg
    t = lg.Throughput(batch_size=2, world_size=4, grad_accum_usteps=3, tp_size=8, model="Mamba7B", seq_length=2048,
                      chip_flops=100.0)
    assert t.seqs_per_iteration == 24
    D, layers, N, L = 4096, 64, 128, 2048
    per_layer = 12 * L * D ** 2 + 8 * L * D + 2 * L * N * D
    want = 3 * per_layer * layers * (2 * 3) / 1e12 / (100.0 * 8)     # fwd + bwd = 3x, per-DP-rank batch, flops of TP chips
    assert abs(t.MFU_factor - want) / want < 1e-12
    step_time, seqs_per_s, mfu = t.get_throughput()
    assert step_time > 0 and abs(seqs_per_s - 24 / step_time) < 1e-6 and abs(mfu - want / step_time) < 1e-9


def test_training_metrics_store_round_trip():
    from state_space_models_neuron_b200.utils.logging import TrainingMetrics
    with tempfile.TemporaryDirectory() as d:
        f = os.path.join(d, "m.json")
        m = TrainingMetrics(f)
        m.update(loss=1.5, step=3)
        m.store_parameters(lr=1e-3, model="Mamba130M")
        again = TrainingMetrics(f)
        assert again.data["metrics"] == {"loss": 1.5, "step": 3} and again.data["parameters"]["model"] == "Mamba130M"
        assert json.load(open(f))["parameters"]["lr"] == "0.001"


def test_debug_helpers():
    from state_space_models_neuron_b200.utils import debug
    buf = debug.CanaryBuffer((4, 8), torch.float32, "cpu", guard_bytes=64)
    buf.tensor.fill_(1.0)
    assert buf.intact()
    buf.raw[10] = 0                     # a write before the tensor is detected
    assert not buf.intact()
    debug.assert_deterministic(lambda x: x * 2, [torch.ones(3)])
    with pytest.raises(AssertionError):
        debug.assert_deterministic(lambda x: x + torch.rand(3), [torch.ones(3)])
    with pytest.raises(FloatingPointError):
        debug.check_finite(torch.tensor([1.0, float("nan")]), "t")
    # the GEMM's rotated tile order still visits every tile once, for the all-gather and reduce-scatter rotations
    assert debug.tile_schedule_is_permutation(16, 10, 8, 132) and debug.tile_schedule_is_permutation(16, 16, 2, 148)


def test_gemm_schedule_covers_every_k_block_once():
    """Property test of the GEMM work distribution (full waves + K-split tail), the host model of the index
    arithmetic in ops/csrc/gemm.cu: the shapes of the training step and a random sweep."""
    from hypothesis import given, settings, strategies as st
    from state_space_models_neuron_b200.utils import debug
    for tiles, units, kb in [(160, 148, 64), (80, 74, 64), (208, 148, 64), (20, 148, 80), (1, 148, 3), (148, 148, 16),
                             (149, 148, 16), (295, 148, 1), (6, 74, 5), (73, 74, 4), (75, 74, 8)]:
        assert debug.gemm_schedule_covers_once(tiles, units, kb), (tiles, units, kb)
        assert debug.gemm_schedule_covers_once(tiles, units, kb, accumulate=True), (tiles, units, kb)
    units, work = debug.gemm_schedule(80, 74, 64)
    assert units == 74 and sum(1 for w in work if w[5] > 1) == 24 and max(w[5] for w in work) == 4

    @settings(max_examples=300, deadline=None)
    @given(st.integers(1, 2000), st.sampled_from([1, 2, 37, 74, 132, 148, 160]), st.integers(1, 300), st.booleans())
    def prop(tiles, units, kb, acc):
        assert debug.gemm_schedule_covers_once(tiles, units, kb, acc)
    prop()


def test_ncu_command_always_leaves_clocks_alone():
    from state_space_models_neuron_b200.utils.profiling import ncu_command
    cmd = ncu_command(["python", "bench.py", "--small"], "gemm_bf16", launches=2, skip=1, out="x/prof")
    assert cmd[:3] == ["ncu", "--clock-control", "none"] and cmd[-3:] == ["python", "bench.py", "--small"]
    assert "regex:gemm_bf16" in cmd and cmd[cmd.index("-c") + 1] == "2" and cmd[cmd.index("-s") + 1] == "1"
    light = ncu_command(["python", "x.py"], None, full=False)
    assert "gpu__time_duration.sum" in light and "--set" not in light


def test_fused_sequence_numbers_advance_on_their_own(monkeypatch):
    """Gradient accumulation makes far more than 65536 fused collective calls between optimizer steps: the
    workspace starts a new block of sequence numbers by itself instead of failing, at the same call on every rank.
    Buffer parity alternates per kind and is not reset when a new block starts."""
    from state_space_models_neuron_b200.ops import cuda_ops
    from state_space_models_neuron_b200.parallel import symm
    launched = []
    monkeypatch.setattr(cuda_ops, "_run", lambda name, *a: launched.append((name, a[1])))
    monkeypatch.setattr(cuda_ops, "_st", lambda: None)
    ws = symm.SymmWorkspace.__new__(symm.SymmWorkspace)
    symm.SeqCounter.__init__(ws)
    ws.seq_base, ws.base_ptrs, ws.me = torch.zeros(1, dtype=torch.int32), [0], 0
    got = [ws.next_seq(symm.KIND_AG if i % 3 else symm.KIND_RS) for i in range(150000)]
    positions = [s for s, _ in got]
    assert min(positions) == 1 and max(positions) < symm.SymmWorkspace.STEP_STRIDE
    assert [n for n, _ in launched] == ["ssm_advance_counter"] * 2 and all(s == symm.SymmWorkspace.STEP_STRIDE for _, s in launched)
    for kind in (symm.KIND_AG, symm.KIND_RS):
        pars = [p for i, (_, p) in enumerate(got) if (symm.KIND_AG if i % 3 else symm.KIND_RS) == kind]
        assert pars[:4] == [0, 1, 0, 1] and all(a != b for a, b in zip(pars, pars[1:]))
    last_par = ws.kind_calls[symm.KIND_AG] & 1
    ws.advance_step()
    assert ws.seq == 0 and ws.next_seq(symm.KIND_AG) == (1, last_par)
    ws.next_seq(symm.KIND_AG)
    ws.next_seq(symm.KIND_AG)
    ws.advance_step(compact=True)
    assert launched[-1] == ("ssm_advance_counter", 4)          # 3 calls -> next even number above them


def test_sequence_compare_is_wrap_safe():
    """The kernels decide "flag has reached seq" by the signed 32-bit distance.  Model of that arithmetic: it holds
    across the wrap from 2^31 - 1 to -2^31 and for every gap below 2^31; a flag that lags more than 2^29 behind is
    pulled up to the base when the base crosses a multiple of 2^29, and a base value never satisfies a wait of its
    own block."""
    def i32(x):
        return (x + 2 ** 31) % 2 ** 32 - 2 ** 31

    def reached(flag, seq):
        return i32(flag - seq) >= 0

    for base in (0, 2 ** 31 - 70000, 2 ** 31 - 3, -2 ** 31 + 5, -70000, 2 ** 32 - 10):
        for pos in (1, 2, 65533):
            seq = i32(base + pos)
            assert reached(seq, seq) and reached(i32(seq + 1), seq) and reached(i32(seq + 65536 * 3), seq)
            assert not reached(i32(seq - 1), seq) and not reached(i32(base), seq)
            assert not reached(i32(seq - 65536 * 1000), seq)

    def advance(base, stride, flags):             # advance_counter_kernel
        old, new = base % 2 ** 32, (base + stride) % 2 ** 32
        if (old >> 29) != (new >> 29):
            flags = [i32(new) if i32(new - f) > 2 ** 29 else f for f in flags]
        return i32(new), flags

    base, flags = 0, [0, 0]                      # flag 0 is in use every step, flag 1 never
    for step in range(70000):                    # more than one full trip around the 32-bit range
        seq = i32(base + 7)
        assert not reached(flags[1], seq), step   # an idle flag must never look "arrived"
        flags[0] = seq
        base, flags = advance(base, 65536, flags)


def test_replay_safety_check():
    from state_space_models_neuron_b200.parallel import symm
    AG, RS, AR = symm.KIND_AG, symm.KIND_RS, symm.KIND_AR
    c = symm.SeqCounter()
    c.recording = []
    for k in (AG, RS, RS, AG, RS, AG, AR):               # odd counts per kind, other collectives in between
        c.take(k)
    rec = c.recording
    assert rec[0] == (AG, 0) and rec[3] == (AG, 1) and rec[5] == (AG, 0)
    symm.check_replay_safe(rec + rec)
    symm.check_replay_safe([(AG, 0), (AG, 1)] * 2)         # alternating buffers back to back are fine
    with pytest.raises(RuntimeError):
        symm.check_replay_safe([(AG, 0)] * 2)              # the same buffer back to back across replays
    with pytest.raises(RuntimeError):
        symm.check_replay_safe([(RS, 1), (AG, 0), (AG, 1), (AG, 1)])


def test_symmetric_workspace_regions_do_not_overlap():
    """Byte layout of the peer-mapped workspace: flags, 2 gather buffers, 2 landing zones, small all-reduce slots and
    2 embedding buffers are disjoint, ordered and inside the allocation, for several TP sizes."""
    from state_space_models_neuron_b200.parallel import symm
    for nranks, rows, cols in [(2, 2048, 4096), (8, 2048, 4096), (4, 4096, 4096), (8, 64 * 8, 2560)]:
        ws = symm.SymmWorkspace.__new__(symm.SymmWorkspace)
        ws.nranks, ws.rows_total, ws.cols = nranks, rows, cols
        elems = rows * cols
        ws.gather_bytes, ws.flags_bytes = (elems * 2 + 1023) // 1024 * 1024, 4096
        ws.slots_bytes = 2 * symm.MAX_RANKS * symm.SMALL_N_MAX * 4
        ws.embed_bytes = (-(-elems // nranks) * 2 + 1023) // 1024 * 1024
        total = ws.flags_bytes + 4 * ws.gather_bytes + ws.slots_bytes + 2 * ws.embed_bytes
        regions = [(0, ws.flags_bytes)]
        regions += [(ws.gather_offset(p), ws.gather_bytes) for p in (0, 1)]
        regions += [(ws.land_offset(p), ws.gather_bytes) for p in (0, 1)]
        regions += [(ws.slots_offset(p), symm.MAX_RANKS * symm.SMALL_N_MAX * 4) for p in (0, 1)]
        regions += [(ws.embed_offset(p), ws.embed_bytes) for p in (0, 1)]
        end = 0
        for off, size in regions:
            assert off >= end and off % 16 == 0, (nranks, off, end)
            end = off + size
        assert end <= total
        # flag words of the four kinds x two parities x (eight sources x four row groups) fit in the flag page
        assert ws.flag_base(symm.KIND_EMB, 1) + symm.FLAG_SLOTS == symm.N_FLAGS <= ws.flags_bytes // 4


def test_fused_tuner_picks_the_fastest_combination_and_leaves_it_switched_on(monkeypatch):
    """`fused_tune.pick_fastest` with scripted step times: chooses the minimum, frees every candidate before the
    next is built, rebuilds the winner, and leaves the two kernel switches on the choice."""
    from state_space_models_neuron_b200.parallel import fused, fused_tune
    script = {(True, True): 50.0, (False, True): 41.0, (True, False): 47.0, (False, False): 43.0}
    built, released, alive = [], [], [0]

    def build():
        key = (fused.kernel_enabled("ag_gemm"), fused.kernel_enabled("gemm_rs"))
        built.append(key)
        alive[0] += 1
        assert alive[0] == 1, "two captured steps alive at once"
        step = lambda: None
        step.key = key
        return step

    def release(step):
        released.append(step.key)
        alive[0] -= 1

    monkeypatch.setattr(fused_tune, "time_steps", lambda run, reps, device: script[run.key])
    before = fused.kernels()
    try:
        rep = fused_tune.pick_fastest(build, "cpu", reps=2, release=release)
        assert rep["chosen"] == "ag_gemm=nccl,gemm_rs=fused"
        assert rep["step"].key == (False, True)
        assert built == list(fused_tune.COMBOS) + [(False, True)] and released == list(fused_tune.COMBOS)
        assert fused.kernels() == {"ag_gemm": False, "gemm_rs": True}
        assert rep["ms"]["ag_gemm=fused,gemm_rs=fused"] == 50.0
        # a combination that cannot be built is skipped
        alive[0] = 0
        calls = [0]

        def build_some():
            calls[0] += 1
            return None if calls[0] == 1 else build()
        rep = fused_tune.pick_fastest(build_some, "cpu", release=release)
        assert rep["ms"]["ag_gemm=fused,gemm_rs=fused"] is None and rep["chosen"] == "ag_gemm=nccl,gemm_rs=fused"
        # a failed health check stops the tuner (the candidate is released first)
        alive[0] = 0
        released.clear()
        checks = iter([True, False])
        with pytest.raises(fused_tune.CandidateFailed):
            fused_tune.pick_fastest(build, "cpu", release=release, healthy=lambda: next(checks))
        assert released == list(fused_tune.COMBOS[:2]) and alive[0] == 0
    finally:
        for k, v in before.items():
            fused.set_kernel(k, v)


def test_native_gemm_plan_matches_the_host_model_and_covers_every_tile_once():
    """The tiling / K-split plan computed by the native library (host code, no GPU needed) agrees with the Python
    model of the schedule in utils/debug.py, and the resulting work list computes every (tile, k-block) exactly once."""
    from state_space_models_neuron_b200.ops import native
    from state_space_models_neuron_b200.utils import debug
    try:
        native.lib()
    except Exception as e:                                   # no nvcc / library on this machine
        pytest.skip(f"native library not available: {e}")
    shapes = [(2048, 18560, 4096), (2048, 2320, 4096), (2320, 4096, 2048), (64, 2560, 5120), (2048, 1024, 4096),
              (18560, 4096, 2048), (2048, 4096, 1024), (128, 128, 64), (300, 6286, 1032), (2048, 50288, 4096),
              (8192, 8192, 8192), (1, 2560, 5120), (4096, 1024, 2048)]
    for M, N, K in shapes:
        for accumulate in (False, True):
            for allow_pair in (True, False):
                plan = debug.gemm_plan(M, N, K, accumulate=accumulate, allow_pair=allow_pair)
                pair = bool(plan["pair"])
                assert plan["bn"] in (128, 192, 256) and (allow_pair or not pair) and (M > 128 or not pair)
                tile_m = 256 if pair else 128
                assert plan["tiles_m"] == -(-M // tile_m) and plan["tiles_n"] == -(-N // plan["bn"])
                tiles = plan["tiles_m"] * plan["tiles_n"]
                max_units = 74 if pair else 148
                kblocks = -(-K // 64)
                units, work = debug.gemm_schedule(tiles, max_units, kblocks, accumulate=accumulate, pair=pair,
                                                  cost_kb=debug.gemm_tile_cost_kb(plan["bn"], pair), always_split=False)
                assert units == plan["units"], (M, N, K, accumulate, allow_pair, plan, units)
                splits = {w[5] for w in work if w[5] > 1} or {1}
                assert splits == {plan["split"]}, (M, N, K, plan, splits)
                assert plan["full_tiles"] + plan["rem"] == tiles and plan["rem"] * plan["split"] <= max(units, 1)
                # every (tile, k-block) exactly once
                seen = {}
                for _, tile, kb0, kb1, sl, ns in work:
                    assert kb1 > kb0
                    for kb in range(kb0, kb1):
                        assert (tile, kb) not in seen
                        seen[(tile, kb)] = 1
                assert len(seen) == tiles * kblocks


def test_all_gather_push_boxes_cover_the_shard_once_and_evenly():
    """Model of the shard push of the all-gather GEMM: for the shard sizes of TP = 2, 4, 8 (and odd widths) every
    64-column x push_rows box is moved by exactly one CTA, groups go out in column order, and no CTA moves more than
    one box more than another."""
    from state_space_models_neuron_b200.utils import debug
    for rows, K, grid in [(1024, 4096, 148), (512, 4096, 148), (256, 4096, 148), (256, 4096, 74), (128, 520, 148),
                          (2048, 1032, 148), (256, 8192, 148), (128, 64, 16)]:
        push_rows, col_blocks, group_kb, ngroups, nslots = debug.ag_push_plan(rows, K)
        assert push_rows in (32, 64, 128) and rows % push_rows == 0 and 1 <= ngroups <= 4 and nslots in (2, 4, 8)
        per_cta = debug.ag_push_boxes(grid, rows, push_rows, col_blocks, group_kb)
        seen = {}
        for boxes in per_cta:
            assert [b[0] for b in boxes] == sorted(b[0] for b in boxes)          # group by group
            for g, row, col in boxes:
                assert (row, col) not in seen and col // 64 // group_kb == g and row < rows and col < col_blocks * 64
                seen[(row, col)] = g
        assert len(seen) == (rows // push_rows) * col_blocks
        counts = [len(b) for b in per_cta]
        assert max(counts) - min(counts) <= 1
    # the sizes the model step uses: 32-row boxes and eight staging slots at TP=8, one box per CTA and group
    assert debug.ag_push_plan(256, 4096)[0] == 32 and debug.ag_push_plan(256, 4096)[4] == 8
    assert debug.ag_push_plan(512, 4096)[0] == 64 and debug.ag_push_plan(1024, 4096)[0] == 128
