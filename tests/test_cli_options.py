"""The command line's option checks (no device needed): what it refuses, it refuses before loading anything."""
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_option_errors_are_said_before_anything_is_loaded():
    for options in (["--preset", "tiny-a"], ["--model-id", "x", "--preset", "tiny-a", "--random-weights"], []):
        proc = subprocess.run([sys.executable, "-m", "qwen_triton_b200.scripts.smoke", *options, "--prompt-ids", "1"], cwd=ROOT,
                              capture_output=True, text=True, timeout=300)
        assert proc.returncode == 2 and "--model-id FOLDER or --preset NAME --random-weights" in proc.stderr
    proc = subprocess.run([sys.executable, "-m", "qwen_triton_b200.scripts.smoke", "--preset", "tiny-a", "--random-weights",
                           "--prompt-ids", "1", "--random-prompts", "4"], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 2 and "one of --prompt, --prompt-ids and --random-prompts" in proc.stderr
