"""train.py end to end on CPU: synthetic data, periodic checkpoints, exact resume."""
import os
import re
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LOG = re.compile(r"step: (\d+), step_loss : ([0-9.]+) learning_rate : ([0-9.e+-]+)")


def _train(d, *extra):
    cmd = [sys.executable, os.path.join(ROOT, "train.py"), "--model", "Mamba130M", "--vocab_size", "512", "--seq_len", "128",
           "--batch", "1", "--synthetic_data", "--dtype", "float32", "--device", "cpu", "--head_dim", "64", "--n_groups", "1",
           "--warmup_steps", "2", "--lr", "1e-3", "--logging_interval", "1", "--checkpoint_dir", os.path.join(d, "ck"),
           "--output_dir", os.path.join(d, "tb"), "--tag", "t", *extra]
    env = dict(os.environ, OMP_NUM_THREADS="4")
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return {int(s): (float(l), float(lr)) for s, l, lr in LOG.findall(r.stdout)}, r.stdout


def test_train_checkpoint_and_exact_resume():
    with tempfile.TemporaryDirectory() as d:
        full, _ = _train(d, "--max_steps", "4", "--checkpoint_freq", "2")
        assert sorted(full) == [1, 2, 3, 4]
        assert os.path.isdir(os.path.join(d, "ck", "t_step_2")) and os.path.isdir(os.path.join(d, "ck", "t_step_4"))
        resumed, out = _train(d, "--max_steps", "4", "--resume", "--checkpoint_load_dir", os.path.join(d, "ck"),
                              "--checkpoint_load_tag", "t_step_2")
        assert "(step 2)" in out
        assert sorted(resumed) == [3, 4]
        for s in (3, 4):                                    # same batches, same optimizer state, same schedule
            assert abs(resumed[s][0] - full[s][0]) < 2e-4, (s, resumed[s], full[s])
            assert abs(resumed[s][1] - full[s][1]) < 1e-9, (s, resumed[s], full[s])
