"""The training entry script end to end on CPU: a synthetic run, then a second start with the same experiment name that
``auto_resume`` continues from the first run's latest checkpoint."""
import importlib.util
import json
import os

import torch


def _main_module():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "Main.py")
    spec = importlib.util.spec_from_file_location("main_entry", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_main_trains_and_auto_resumes(tmp_path):
    main = _main_module()
    args = ["--preset", "tiny_cpu", "--synthetic", "16", "--no-orchestrator", "--override", f"output_dir={tmp_path}",
            "experiment_name=entry", "num_epochs=1", "num_layers=2", "hidden_size=64", "num_heads=4", "num_kv_heads=2",
            "intermediate_size=128", "seq_length=32", "vocab_size=512", "num_workers=0", "auto_epoch_scaling=False"]
    assert main.main(args) == 0
    exp = os.path.join(str(tmp_path), "entry")
    ck_dir = os.path.join(exp, "checkpoints")
    assert os.path.exists(os.path.join(ck_dir, "checkpoint_final.pt"))
    with open(os.path.join(exp, "training_summary.json")) as f:
        first = json.load(f)
    steps_first = torch.load(os.path.join(ck_dir, "checkpoint_final.pt"), weights_only=False)["global_step"]
    assert steps_first == 4 and first
    # second start, same experiment: continues at step 4 instead of starting over
    assert main.main(args) == 0
    steps_second = torch.load(os.path.join(ck_dir, "checkpoint_final.pt"), weights_only=False)["global_step"]
    assert steps_second > steps_first
    # auto_resume off: starts from step 0 again
    assert main.main(args + ["auto_resume=False"]) == 0
    assert torch.load(os.path.join(ck_dir, "checkpoint_final.pt"), weights_only=False)["global_step"] == steps_first
