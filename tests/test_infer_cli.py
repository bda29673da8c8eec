"""The generation driver: same flags and error behaviour as the reference's infer.py (289-357),
run on a config-built model because no checkpoint is available offline."""
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from kuillm_b200 import infer  # noqa: E402


def test_flags_match_the_reference_driver():
    opts = {a.dest for a in infer.build_parser()._actions}
    for name in ("prompt", "prompts", "batch", "max_new_tokens", "temperature", "show", "use_kuiper", "timing", "verify", "verify_tol"):
        assert name in opts


def test_conflicting_flags_are_refused(tmp_path):
    f = tmp_path / "p.txt"
    f.write_text("a\nb\n")
    with pytest.raises(SystemExit):
        infer.main(["hello", "--prompts", str(f), "--shape", "tiny", "--device", "cpu"])
    with pytest.raises(SystemExit):
        infer.main(["--verify", "--no-kuiper", "--shape", "tiny", "--device", "cpu"])
    empty = tmp_path / "e.txt"
    empty.write_text("\n")
    assert infer.main(["--prompts", str(empty), "--shape", "tiny", "--device", "cpu"]) == 1


def test_cpu_generation_without_kernels(capsys, tmp_path):
    f = tmp_path / "p.txt"
    f.write_text("first prompt\nsecond, longer prompt\nthird\n")
    rc = infer.main(["--prompts", str(f), "--shape", "tiny", "--device", "cpu", "--dtype", "float32", "--batch", "2",
                     "--max-new-tokens", "3", "--temperature", "0", "--timing", "--print"])
    out = capsys.readouterr().out
    assert rc == 0
    assert "[batched generate / torch] 3 prompts (padded to 4), 3 new tokens each" in out
    assert "[timing] prefill" in out and out.count("Response:") == 3


@pytest.mark.gpu
def test_gpu_generation_dispatches_and_verifies(capsys):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    rc = infer.main(["a prompt", "--shape", "tiny", "--batch", "4", "--max-new-tokens", "6", "--temperature", "0", "--verify"])
    out = capsys.readouterr().out
    assert "[batched generate / kuiper+verify] 1 prompts (padded to 4), 6 new tokens each" in out
    assert "[verify] result: PASS" in out and rc == 0
