"""The user-facing pages stay true to the package: their Python examples compile and name attributes that exist, the
environment variables they list are read somewhere, every variable of the configuration is listed, and the quick
start of the front page trains on the CPU path."""
import glob
import os
import re
import tempfile

import torch

import tensornet_b200 as tn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PAGES = [os.path.join(ROOT, "README.md")] + sorted(glob.glob(os.path.join(ROOT, "docs", "*.md")))
KNOB = re.compile(r"TN_[A-Z0-9_]*[A-Z0-9]")


def _python_blocks(path):
    with open(path) as f:
        return re.findall(r"```python\n(.*?)```", f.read(), re.S)


def _source_text():
    out = []
    for pat in ("tensornet_b200/**/*.py", "tensornet_b200/csrc/*", "bench.py", "benchmarks/*.py", ".github/workflows/*.yml"):
        for p in glob.glob(os.path.join(ROOT, pat), recursive=True):
            if os.path.isfile(p) and not p.endswith((".so", ".o")):
                with open(p, errors="ignore") as f:
                    out.append(f.read())
    return "\n".join(out)


def test_python_examples_compile_and_name_real_attributes():
    seen = 0
    for page in PAGES:
        for block in _python_blocks(page):
            compile(block, page, "exec")
            for dotted in set(re.findall(r"\btn((?:\.[A-Za-z_][A-Za-z_0-9]*)+)", block)):
                obj = tn
                for part in dotted.strip(".").split("."):
                    assert hasattr(obj, part), f"{page}: tn{dotted} does not exist"
                    obj = getattr(obj, part)
                seen += 1
            for mod, names in re.findall(r"^from (tensornet_b200[.\w]*) import (.+)$", block, re.M):
                m = __import__(mod, fromlist=["_"])
                for n in names.split(","):
                    assert hasattr(m, n.strip()), f"{page}: {mod}.{n.strip()} does not exist"
                    seen += 1
    assert seen >= 10


def test_every_documented_variable_is_read_and_every_config_variable_is_documented():
    src = _source_text()
    with open(PAGES[0]) as f:
        readme = f.read()
    for page in PAGES:
        with open(page) as f:
            for k in set(KNOB.findall(f.read())):
                if k in ("TN_GEMM",):          # prefix of a family named with a wildcard
                    continue
                assert k in src, f"{page} names {k}, which nothing reads"
    with open(os.path.join(ROOT, "tensornet_b200", "core", "config.py")) as f:
        for k in set(re.findall(r'_env\("(TN_[A-Z0-9_]+)"', f.read())):
            assert f"`{k}`" in readme, f"{k} is read by the configuration but missing from the front page's table"


def test_front_page_quick_start_trains_on_the_cpu_path():
    block = _python_blocks(PAGES[0])[0]
    slots = [str(i) for i in range(1, 27)]
    g = torch.Generator().manual_seed(0)

    def batch():
        f = {s: torch.randint(1, 1000, (32,), generator=g) for s in slots}
        f["dense"] = torch.randn(32, 13, generator=g)
        return f, (torch.rand(32, generator=g) < 0.3).float()

    with tempfile.TemporaryDirectory() as d:
        code = block.replace('"/data/model"', repr(d))
        assert repr(d) in code
        env = {"dataset": [batch() for _ in range(3)]}
        exec(compile(code, "README.md", "exec"), env)
        assert os.path.isdir(os.path.join(d, "2024-01-01"))
        model = env["model"]
        p = model.predict_on_batch(env["dataset"][0][0])
        assert p.shape[0] == 32 and bool(torch.isfinite(p).all())
