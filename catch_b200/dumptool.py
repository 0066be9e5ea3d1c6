"""Op-level tensor dump tool (reference: torch_mlu/core/dumptool.py:34-91).

    with Dumper("./dump", enable=True, use_cpu=True, level=2):
        y = model(x)

Every operator that touches a device tensor gets a directory ``<k>_<op>`` (nested for
ops called inside ops) with ``dev_<i>`` files for its tensor arguments and
``dev_result_<i>`` for its results; with ``use_cpu`` the operator is also re-run on CPU
copies of the arguments and ``cpu_result_<i>`` is written next to the device result.
Level 0 dumps the first 10 values of each tensor, 1 the sum of absolute values, 2 all
values.  An existing directory is never overwritten: the next free ``<dir><N>`` is used.

``dump_gencase(enable, level)`` is the kernel case generator (reference:
``dump_cnnl_gencase``, torch_mlu/core/dumptool.py:34-73): while it is on, every operator
that touches a device tensor writes a JSON description of the call under ``./gen_case``
(level ``"L1"``), with the tensor bytes (``"L2"``) or to the screen (``"L3"``);
``replay_case`` re-runs such a file on the device and on the CPU.
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


_GENCASE_LEVELS = ("L1", "L2", "L3")


def dump_gencase(enable: bool = True, level: str = "L1", case_dir: str = "./gen_case") -> bool:
    """Turn the kernel case generator on or off; returns its new state.

    ``"L1"``: dtype, shape, stride, memory format of every tensor argument and the value of every other argument, one
    JSON file per call under ``<case_dir>/<op>/``.  ``"L2"``: also the bytes of the tensor arguments (slow).
    ``"L3"``: the same description printed to stderr, no files.  When the environment variable ``CATCH_B200_GEN_CASE``
    is set the generator is controlled from there (it is switched on at import) and this call warns and does nothing,
    as the reference does for ``CNNL_GEN_CASE``."""
    import os
    import warnings

    if os.environ.get("CATCH_B200_GEN_CASE") is not None:
        warnings.warn("unset the environment variable 'CATCH_B200_GEN_CASE', or dump_gencase() will not work")
        return False
    if not enable:
        _C._dump_gencase(0)
        return False
    if level not in _GENCASE_LEVELS:
        raise ValueError(f"dump_gencase only supports the levels 'L1', 'L2' and 'L3', got {level!r}")
    _C._dump_gencase(_GENCASE_LEVELS.index(level) + 1, case_dir)
    return True


def _gencase_from_env() -> None:
    import os

    v = os.environ.get("CATCH_B200_GEN_CASE")
    if v in ("1", "2", "3"):
        _C._dump_gencase(int(v), os.environ.get("CATCH_B200_GEN_CASE_DIR", "./gen_case"))


_gencase_from_env()


def replay_case(path: str, device: str = "blackwell", seed: int = 0):
    """Re-run one case file: returns ``(device_results, cpu_results, errors)``, ``errors`` being the relative RMS error
    of every floating-point result.  Tensors come from the ``.bin`` files of a level-2 case, else they are random
    (normal for floating types, small non-negative integers otherwise) with the recorded dtype, shape and strides."""
    import json
    import os

    import torch

    with open(path) as f:
        case = json.load(f)
    ns, _, rest = case["op"].partition("::")
    name, _, overload = rest.partition(".")
    op = getattr(getattr(getattr(torch.ops, ns), name), overload or "default")
    gen = torch.Generator().manual_seed(seed)
    base = os.path.dirname(os.path.abspath(path))
    dtypes = {str(d).split(".")[-1].lower(): d for d in (
        torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8, torch.uint8, torch.int16, torch.int32,
        torch.int64, torch.bool)}
    names = {"float": "float32", "double": "float64", "half": "float16", "char": "int8", "byte": "uint8",
             "short": "int16", "int": "int32", "long": "int64"}
    # ScalarType / MemoryFormat / Layout arguments are recorded as their integer codes
    scalar_types = [torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64, torch.float16, torch.float32,
                    torch.float64, None, None, None, torch.bool, None, None, None, torch.bfloat16]
    formats = [torch.contiguous_format, torch.preserve_format, torch.channels_last, torch.channels_last_3d]

    def tensor(d):
        key = d["dtype"].lower()
        dt = dtypes[names.get(key, key)]
        shape, stride = d["shape"], d["stride"]
        span = 1 + sum((n - 1) * s for n, s in zip(shape, stride)) if all(n > 0 for n in shape) else 0
        if "data" in d:
            flat = torch.frombuffer(bytearray(open(os.path.join(base, d["data"]), "rb").read()), dtype=dt).reshape(shape)
            t = torch.empty(span, dtype=dt).as_strided(shape, stride)
            t.copy_(flat)
        elif dt.is_floating_point:
            t = torch.randn(span, generator=gen).to(dt).as_strided(shape, stride)
        elif dt == torch.bool:
            t = (torch.rand(span, generator=gen) > 0.5).as_strided(shape, stride)
        else:
            t = torch.randint(0, 2, (span,), generator=gen).to(dt).as_strided(shape, stride)
        return t.requires_grad_(True) if d.get("requires_grad") and dt.is_floating_point else t

    def value(d, want_device):
        k = d["kind"]
        if k == "tensor":
            t = tensor(d)
            if want_device and d["device"] == "device":
                moved = torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=device)
                moved.copy_(t.detach())
                return moved.requires_grad_(t.requires_grad)
            return t
        if k == "none":
            return None
        if k == "float":
            return float(d["value"])
        if k == "float_list":
            return [float(x) for x in d["value"]]
        if k == "bool_list":
            return [bool(x) for x in d["value"]]
        if k in ("tensor_list", "list"):
            return [value(e, want_device) for e in d["value"]]
        if k == "device":
            return torch.device(device if want_device and d["value"] == "device" else "cpu")
        if k == "int":
            ty = d.get("type", "")
            if "ScalarType" in ty:
                return scalar_types[d["value"]]
            if "MemoryFormat" in ty:
                return formats[d["value"]]
            if "Layout" in ty:
                return torch.strided
            return d["value"]
        if k in ("bool", "string", "int_list"):
            return d["value"]
        raise ValueError(f"replay_case: argument {d.get('name')} of kind {k} ({d.get('tag')}) cannot be rebuilt")

    def run(want_device):
        gen.manual_seed(seed)
        args, kwargs = [], {}
        schema_args = op._schema.arguments
        for d, a in zip(case["args"], schema_args):
            v = value(d, want_device)
            if a.kwarg_only:
                kwargs[a.name] = v
            else:
                args.append(v)
        out = op(*args, **kwargs)
        return list(out) if isinstance(out, (tuple, list)) else [out]

    dev_out, cpu_out = run(True), run(False)
    errors = []
    for a, b in zip(dev_out, cpu_out):
        if isinstance(a, torch.Tensor) and a.is_floating_point():
            x, y = a.detach().cpu().double(), b.detach().double()
            errors.append(float((x - y).norm() / (y.norm() + 1e-12)))
        else:
            errors.append(None)
    return dev_out, cpu_out, errors


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
