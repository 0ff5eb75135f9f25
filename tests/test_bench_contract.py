"""What the measurement script promises without a GPU: more than one GPU is refused with one line and
exit code 2; the reference arm prints one JSON line, either a result or why it is unavailable; the size
tables hold the three model sizes with the keys the architecture's configuration needs."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=300, env=e, cwd=ROOT)


def test_more_than_one_gpu_is_refused_with_one_line():
    r = _run("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout
    # launched as ranks of a larger job: only rank 0 speaks
    r = _run("--gpus", "2", env={"WORLD_SIZE": "2", "RANK": "1"})
    assert r.returncode == 2 and r.stdout.strip() == ""


def test_reference_arm_prints_one_json_line():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    lines = r.stdout.strip().splitlines()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and ("unavailable" in d or "value" in d)
    if "unavailable" in d:
        assert "\n" not in d["unavailable"] and len(d["unavailable"]) > 10


def test_size_tables_parse_as_configurations():
    from atom_b200.benchmarks.sizes import SIZES
    from atom_b200.config import config_from_dict
    assert set(SIZES) == {"4b", "8b", "32b"}
    for name, (cfg, seed) in SIZES.items():
        c = config_from_dict(dict(cfg))
        assert c.architecture == "Qwen3ForCausalLM" and isinstance(seed, int)
    assert SIZES["4b"][0]["tie_word_embeddings"] and not SIZES["8b"][0]["tie_word_embeddings"]
    assert SIZES["32b"][0]["num_hidden_layers"] == 64 and SIZES["32b"][0]["num_attention_heads"] == 64
