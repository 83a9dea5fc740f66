"""Every `python bench.py ...` command that a summary under profiles/ quotes must still be a command bench.py accepts: the
summaries promise that they can be reproduced from committed files."""
import glob
import os
import re
import shlex
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def quoted_commands():
    out = []
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        for line in open(path, encoding="utf-8"):
            m = re.search(r"python bench\.py([^`\n]*)", line)
            if not m or not line.startswith("    "):      # indented command lines only, not prose that abbreviates with an ellipsis
                continue
            args = m.group(1).split("#")[0].strip()
            if "…" in args or "..." in args:
                continue
            out.append((os.path.basename(path), args))
    return out


def test_there_are_commands_to_check():
    assert len(quoted_commands()) >= 10


@pytest.mark.parametrize("where,args", quoted_commands(), ids=lambda v: v if v.endswith(".md") else None)
def test_quoted_bench_command_parses(where, args, monkeypatch):
    import bench
    monkeypatch.setattr(sys, "argv", ["bench.py", *shlex.split(args)])
    parsed = bench.parse_args()                            # argparse exits with SystemExit(2) on an unknown flag or choice
    if parsed.kernel in ("gemm",):
        assert len(parsed.shape) == 3, where
    if parsed.kernel in ("pack",):
        assert len(parsed.shape) == 6, where
    if parsed.kernel in ("layer",):
        assert len(parsed.shape) in (6, 7), where
    if parsed.kernel == "fconv":
        assert len(parsed.shape) == 1 and 0 <= parsed.shape[0] < len(bench.FCONV_CASES), where
