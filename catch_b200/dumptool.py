"""Op-level tensor dump tool (reference: torch_mlu/core/dumptool.py:34-91).

    with Dumper("./dump", enable=True, use_cpu=True, level=2):
        y = model(x)

Every operator that touches a device tensor gets a directory ``<k>_<op>`` (nested for
ops called inside ops) with ``dev_<i>`` files for its tensor arguments and
``dev_result_<i>`` for its results; with ``use_cpu`` the operator is also re-run on CPU
copies of the arguments and ``cpu_result_<i>`` is written next to the device result.
Level 0 dumps the first 10 values of each tensor, 1 the sum of absolute values, 2 all
values.  An existing directory is never overwritten: the next free ``<dir><N>`` is used.
"""
from __future__ import annotations

from . import _C


def start_dump(dump_dir: str = "./dump", enable: bool = True, use_cpu: bool = False, level: int = 0) -> None:
    if level not in (0, 1, 2):
        raise ValueError("dump level must be 0, 1 or 2")
    _C._dump_start(dump_dir, enable, use_cpu, level)


def end_dump() -> None:
    _C._dump_finish()


class Dumper:
    def __init__(self, dump_dir: str = "./dump", enable: bool = True, use_cpu: bool = False, level: int = 0):
        self.args = (dump_dir, enable, use_cpu, level)

    def __enter__(self):
        start_dump(*self.args)
        return self

    def __exit__(self, *exc):
        end_dump()
        return False


def compare_dump(op_dir: str, prec: float = 3e-3):
    """Relative RMS error between ``dev_result_*`` and ``cpu_result_*`` files of one op directory."""
    import os

    def read(path):
        with open(path) as f:
            lines = f.read().splitlines()
        return [float(v) for v in lines[1:] if v]

    out = {}
    for name in sorted(os.listdir(op_dir)):
        if name.startswith("dev_result_"):
            k = name[len("dev_result_"):]
            cpu = os.path.join(op_dir, "cpu_result_" + k)
            if os.path.exists(cpu):
                a, b = read(os.path.join(op_dir, name)), read(cpu)
                num = sum((x - y) ** 2 for x, y in zip(a, b)) ** 0.5
                den = sum(y * y for y in b) ** 0.5 + 1e-12
                out[k] = num / den
    return out, all(v <= prec for v in out.values())
