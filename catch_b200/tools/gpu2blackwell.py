"""Convert a directory of PyTorch CUDA scripts to run on the ``blackwell`` device.

    python -m catch_b200.tools.gpu2blackwell -i path/to/scripts [-s]

The converted tree is written next to the input as ``<input>_blackwell/`` together
with ``report.md`` listing every edit.  Same job and CLI shape as the reference's
converter (tools/torch_gpu2mlu.py:39-119):

* every non-``.py`` file is copied unchanged;
* after the first ``import torch`` line of a script, ``import catch_b200`` is added;
* ``cuda`` -> ``blackwell`` and ``nccl`` -> ``bwccl`` on every other line;
* ``--strict`` additionally rewrites ``CUDA``, ``gpu`` and ``GPU``.
"""
from __future__ import annotations

import argparse
import os
import re
import shutil
from dataclasses import dataclass, field
from typing import List, Tuple

RULES = [(re.compile("cuda"), "blackwell"), (re.compile("nccl"), "bwccl")]
# Call sites the rewrite cannot make work: they are left as they are and listed in the report.
NEEDS_ATTENTION = [(re.compile(r"\bnn\.DataParallel\("),
                    "nn.DataParallel drives several devices from one process through torch.cuda only: use one process per "
                    "device with DistributedDataParallel (or catch_b200.parallel.FusedDataParallel) on the bwccl backend")]
STRICT_RULES = [(re.compile("CUDA"), "BLACKWELL"), (re.compile("gpu"), "blackwell"), (re.compile("GPU"), "BLACKWELL")]


@dataclass
class Report:
    entries: List[Tuple[str, int, str]] = field(default_factory=list)

    def add(self, path: str, line: int, what: str) -> None:
        self.entries.append((path, line, what))

    def render(self) -> str:
        out = ["# Blackwell PyTorch Model Migration Report", "## Changes", "| No. |  File  |  Description  |",
               "|---|---|---|"]
        for i, (path, line, what) in enumerate(self.entries, 1):
            out.append(f"| {i} | {path}:{line} | {what} |")
        return "\n".join(out) + "\n"


def convert_source(text: str, rel_path: str, strict: bool, report: Report) -> str:
    """Rewrite one script; records each change in ``report``."""
    rules = RULES + (STRICT_RULES if strict else [])
    out = []
    imported = False
    for n, line in enumerate(text.splitlines(keepends=True), 1):
        if not imported and line.strip() == "import torch":
            imported = True
            out.append(line)
            out.append(line.replace("import torch", "import catch_b200"))
            report.add(rel_path, n, 'add "import catch_b200"')
            continue
        for pat, why in NEEDS_ATTENTION:
            if pat.search(line):
                report.add(rel_path, n, "needs attention: " + why)
        new = line
        for pat, repl in rules:
            new = pat.sub(repl, new)
        if new != line:
            report.add(rel_path, n, f'change "{line.strip()}" to "{new.strip()}"')
        out.append(new)
    return "".join(out)


def convert_tree(input_path: str, strict: bool = False) -> Tuple[str, str]:
    """Convert ``input_path``; returns (output directory, report path)."""
    input_path = os.path.abspath(input_path)
    out_path = input_path + "_blackwell"
    os.makedirs(out_path, exist_ok=True)
    report = Report()
    for root, _dirs, files in os.walk(input_path):
        for name in sorted(files):
            src = os.path.join(root, name)
            rel = os.path.relpath(src, input_path)
            dst = os.path.join(out_path, rel)
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            if not name.endswith(".py"):
                try:
                    shutil.copy(src, dst)
                except OSError as e:
                    print("copy error:", src, e)
                continue
            with open(src, "r", encoding="utf-8", errors="surrogateescape") as f:
                text = f.read()
            with open(dst, "w", encoding="utf-8", errors="surrogateescape") as f:
                f.write(convert_source(text, rel, strict, report))
    report_path = os.path.join(out_path, "report.md")
    with open(report_path, "w", encoding="utf-8") as f:
        f.write(report.render())
    return out_path, report_path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--input", "-i", required=True, help="directory with the CUDA scripts")
    ap.add_argument("--strict", "-s", action="store_true", help="also rewrite CUDA / gpu / GPU")
    args = ap.parse_args(argv)
    out_path, report_path = convert_tree(args.input, args.strict)
    print("# Blackwell PyTorch Model Migration Report")
    print("Official PyTorch model scripts: ", os.path.abspath(args.input))
    print("Blackwell PyTorch model scripts: ", out_path)
    print("Migration Report: ", report_path)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
