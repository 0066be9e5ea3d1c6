"""Device against CPU over a few thousand operator calls: element-wise, broadcasting and type promotion, reductions,
softmax, shape and indexing operators, pooling and resampling, normalisation, the GEMM family, convolutions and losses,
each in several dtypes, shapes (0-dim, empty, odd sizes) and layouts (contiguous, channels-last, transposed, strided),
forward and, where it applies, backward.

    python tests/op_sweep.py [--out op_sweep.log]

Nothing is asserted: every mismatch (relative RMS error above the dtype's tolerance, different shape / dtype, a dense
result whose contiguity differs from the CPU's) and every exception is written to the log, one line each, and the
totals are printed.  The CPU fallback and the per-operator try / catch are switched off, so an operator without a
device kernel shows up as an exception instead of silently running on the host (set CATCH_B200_FALLBACK_TO_CPU=1 /
CATCH_B200_OP_TRYCATCH=1 to see the behaviour a user gets)."""
import os, sys, json, traceback, itertools
os.environ.setdefault("CATCH_B200_FALLBACK_TO_CPU", "0")
os.environ.setdefault("CATCH_B200_OP_TRYCATCH", "0")
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch, torch.nn.functional as F
import catch_b200
import catch_b200.ops.capi
DEV = "blackwell"
n_ok = 0
_out = sys.argv[sys.argv.index("--out") + 1] if "--out" in sys.argv else "op_sweep.log"
_log = open(_out, "w")
class _Fails(list):
    def append(self, item):
        super().append(item)
        _log.write(f"{item[0]} :: {item[1]}\n"); _log.flush()
fails = _Fails()
g = torch.Generator().manual_seed(0)

def tol(dt):
    return {torch.float32: 2e-4, torch.bfloat16: 3e-2, torch.float16: 6e-3, torch.float64: 1e-6}.get(dt, 0)

def to_dev(t):
    if not isinstance(t, torch.Tensor):
        return t
    if t.numel() == 0 or t.dim() == 0:
        return t.detach().to(DEV)
    span = 1 + sum((n - 1) * st for n, st in zip(t.shape, t.stride()))
    base = torch.zeros(span, dtype=t.dtype)
    base.as_strided(t.shape, t.stride()).copy_(t.detach())
    return base.to(DEV).as_strided(t.shape, t.stride())

def cmp(name, a, b, dt):
    if isinstance(a, (tuple, list)):
        return all(cmp(f"{name}[{i}]", x, y, dt) for i, (x, y) in enumerate(zip(a, b)))
    if not isinstance(a, torch.Tensor):
        ok = a == b
        if not ok: fails.append((name, f"value {a} vs {b}"))
        return ok
    a = a.detach().cpu()
    if a.shape != b.shape or a.dtype != b.dtype:
        fails.append((name, f"shape/dtype {tuple(a.shape)} {a.dtype} vs {tuple(b.shape)} {b.dtype}")); return False
    if a.numel() == 0: return True
    dense = b.numel() == 1 + sum((n - 1) * st for n, st in zip(b.shape, b.stride()))  # a view with gaps is moved densely
    if a.dim() >= 2 and dense and a.is_contiguous() != b.is_contiguous() and ".grad" not in name:
        fails.append((name, f"LAYOUT device strides {a.stride()} vs cpu {b.stride()}"))
    if a.dtype.is_floating_point:
        x, y = a.double(), b.detach().double()
        if not torch.equal(torch.isnan(x), torch.isnan(y)):
            fails.append((name, "nan positions")); return False
        x, y = torch.nan_to_num(x, 0, 1e30, -1e30), torch.nan_to_num(y, 0, 1e30, -1e30)
        err = float((x - y).norm() / (y.norm() + 1e-6))
        mx = float((x - y).abs().max() / (y.abs().max() + 1e-6))
        t = tol(b.dtype)
        if b.dtype == torch.float32 and name.split("/")[0] in ("mm", "mm_tn", "addmm", "linear", "bmm", "baddbmm", "matmul_bcast", "matmul_vec", "dot", "linear.grad0"):
            t = 3e-3
        if ".grad" in name and b.dtype == torch.float32 and name.split("/")[0] in ("mm", "linear", "bmm"):
            t = 3e-3
        if err > t or mx > 8 * t:
            fails.append((name, f"rel rms {err:.3e} max {mx:.3e} tol {t}")); return False
        return True
    if not torch.equal(a, b.detach()):
        fails.append((name, f"exact mismatch {(a != b).sum().item()} of {a.numel()}")); return False
    return True

def run(name, fn, args, dt, grad=False):
    global n_ok
    try:
        cargs = [x.detach().clone().requires_grad_(grad and x.dtype.is_floating_point) if isinstance(x, torch.Tensor) else x for x in args]
        dargs = [to_dev(x).requires_grad_(grad and x.dtype.is_floating_point) if isinstance(x, torch.Tensor) else x for x in args]
        ref = fn(*cargs)
        out = fn(*dargs)
        ok = cmp(name, out, ref, dt)
        if grad and ok:
            r0 = ref[0] if isinstance(ref, (tuple, list)) else ref
            o0 = out[0] if isinstance(out, (tuple, list)) else out
            if r0.dtype.is_floating_point and r0.requires_grad:
                w = torch.randn(r0.shape, generator=g).to(r0.dtype)
                r0.backward(w); o0.backward(w.to(DEV))
                for i, (c, d) in enumerate(zip(cargs, dargs)):
                    if isinstance(c, torch.Tensor) and c.requires_grad:
                        if d.grad is None:
                            fails.append((f"{name}.grad{i}", "missing")); ok = False
                        else:
                            ok = cmp(f"{name}.grad{i}", d.grad, c.grad, dt) and ok
        n_ok += bool(ok)
    except Exception as e:  # noqa
        fails.append((name, "EXC " + repr(e)[:300]))

def rnd(shape, dt, pos=False):
    if dt.is_floating_point:
        t = torch.randn(shape, generator=g)
        if pos: t = t.abs() + 0.5
        return t.to(dt)
    if dt == torch.bool:
        return torch.rand(shape, generator=g) > 0.5
    return torch.randint(-5, 6, shape, generator=g).to(dt)

def layouts(shape, dt, pos=False):
    yield "c", rnd(shape, dt, pos)
    if len(shape) == 4:
        yield "cl", rnd(shape, dt, pos).contiguous(memory_format=torch.channels_last)
    if len(shape) >= 2:
        yield "t", rnd(shape[::-1], dt, pos).permute(*range(len(shape))[::-1])
    if len(shape) >= 1 and shape[-1] > 1:
        big = rnd(shape[:-1] + (shape[-1] * 2,), dt, pos)
        yield "s", big[..., ::2]

SHAPES = [(), (1,), (7,), (3, 5), (2, 3, 4, 5), (0, 4), (1031, 17), (2, 8, 6, 6)]
FDT = [torch.float32, torch.bfloat16, torch.float16]

# ---- unary
UN = {"relu": torch.relu, "gelu": F.gelu, "sigmoid": torch.sigmoid, "tanh": torch.tanh, "exp": torch.exp, "abs": torch.abs,
      "neg": torch.neg, "floor": torch.floor, "ceil": torch.ceil, "erf": torch.erf, "silu": F.silu, "hardtanh": F.hardtanh,
      "leaky_relu": lambda x: F.leaky_relu(x, 0.1), "softplus": F.softplus, "sign": torch.sign, "cos": torch.cos,
      "sin": torch.sin, "round": torch.round, "trunc": torch.trunc, "sqr": lambda x: x * x, "clamp": lambda x: x.clamp(-0.5, 0.7),
      "elu": F.elu, "hardswish": F.hardswish, "hardsigmoid": F.hardsigmoid, "relu6": F.relu6, "logsigmoid": F.logsigmoid,
      "tanh_gelu": lambda x: F.gelu(x, approximate="tanh"), "isnan": torch.isnan, "logical_not": torch.logical_not}
UNP = {"log": torch.log, "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "reciprocal": torch.reciprocal, "log2": torch.log2, "log1p": torch.log1p}
for nm, fn in list(UN.items()) + list(UNP.items()):
    for dt in FDT:
        for sh in SHAPES:
            for ln, t in layouts(sh, dt, nm in UNP):
                gr = nm in ("relu", "gelu", "sigmoid", "tanh", "silu", "leaky_relu", "softplus", "elu", "hardswish") and dt != torch.float16 and ln in ("c", "cl")
                run(f"{nm}/{dt}/{sh}/{ln}", fn, [t], dt, grad=gr)
# ---- binary with broadcasting / promotion
BI = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div, "maximum": torch.maximum, "minimum": torch.minimum,
      "eq": torch.eq, "lt": torch.lt, "ge": torch.ge, "ne": torch.ne, "atan2": torch.atan2, "fmod": torch.fmod}
PAIRS = [((3, 5), (3, 5)), ((3, 1, 5), (4, 1)), ((2, 3, 4, 5), (5,)), ((2, 3, 4, 5), (1, 3, 1, 1)), ((7,), ()), ((), (7,)), ((0, 4), (4,)), ((1031, 17), (1031, 1))]
for nm, fn in BI.items():
    for da, db in [(torch.float32,) * 2, (torch.bfloat16,) * 2, (torch.float16,) * 2, (torch.float32, torch.bfloat16), (torch.int64, torch.float32), (torch.int64, torch.int64), (torch.int32, torch.int64)]:
        if nm in ("atan2",) and not (da.is_floating_point and db.is_floating_point): continue
        for sa, sb in PAIRS:
            a, b = rnd(sa, da), rnd(sb, db, pos=nm in ("div", "fmod"))
            if nm in ("div", "fmod") and not db.is_floating_point: b = b.abs() + 1
            run(f"{nm}/{da}/{db}/{sa}/{sb}", fn, [a, b], torch.promote_types(da, db))
    for dt in FDT + [torch.int64]:
        if nm in ("maximum", "minimum", "atan2"): continue
        run(f"{nm}/scalar/{dt}", lambda x, fn=fn: fn(x, 2), [rnd((3, 5), dt)], dt)
run("pow/f32", lambda x: x.pow(2.5), [rnd((3, 5), torch.float32, True)], torch.float32)
run("pow/t", torch.pow, [rnd((3, 5), torch.float32, True), rnd((5,), torch.float32)], torch.float32)
run("where", torch.where, [rnd((3, 5), torch.bool), rnd((3, 5), torch.float32), rnd((5,), torch.float32)], torch.float32)
run("addcmul", lambda a, b, c: torch.addcmul(a, b, c, value=0.5), [rnd((3, 5), torch.float32) for _ in range(3)], torch.float32)
run("addcdiv", lambda a, b, c: torch.addcdiv(a, b, c, value=0.5), [rnd((3, 5), torch.float32), rnd((3, 5), torch.float32), rnd((3, 5), torch.float32, True)], torch.float32)
run("lerp", lambda a, b: torch.lerp(a, b, 0.3), [rnd((3, 5), torch.float32) for _ in range(2)], torch.float32)
def inplace_view(x, y):
    x = x.clone(); x[:, ::2].add_(y); x.t().mul_(2.0); return x
run("inplace_views", inplace_view, [rnd((4, 6), torch.float32), rnd((4, 3), torch.float32)], torch.float32)
# ---- reductions
RED = {"sum": torch.sum, "mean": torch.mean, "amax": torch.amax, "amin": torch.amin, "prod": torch.prod, "var": torch.var, "std": torch.std,
       "logsumexp": torch.logsumexp, "norm": lambda x, dim, keepdim=False: torch.linalg.vector_norm(x, 2, dim=dim, keepdim=keepdim)}
for nm, fn in RED.items():
    for dt in [torch.float32, torch.bfloat16]:
        for sh, dims in [((3, 5), [0, 1, (0, 1)]), ((2, 3, 4, 5), [0, 1, -1, (0, 2), (1, 3), (0, 1, 2, 3)]), ((1031, 17), [0, 1]), ((17, 1031), [0, 1]), ((5, 1, 7), [1])]:
            for dim in dims:
                if nm == "prod" and not isinstance(dim, int): continue
                for ln, t in layouts(sh, dt):
                    if nm == "prod": t = (t.float().clamp(-1.2, 1.2)).to(dt)
                    for kd in (False, True):
                        run(f"{nm}/{dt}/{sh}/{dim}/{ln}/{kd}", lambda x, fn=fn, dim=dim, kd=kd: fn(x, dim=dim, keepdim=kd), [t], dt)
for dt in [torch.float32, torch.bfloat16, torch.int64]:
    for sh in [(3, 5), (2, 3, 4, 5), (1031, 17)]:
        t = rnd(sh, dt)
        run(f"sum_all/{dt}/{sh}", torch.sum, [t], dt)
        run(f"max_all/{dt}/{sh}", torch.max, [t], dt)
        run(f"min_all/{dt}/{sh}", torch.min, [t], dt)
        for dim in range(len(sh)):
            tt = torch.randperm(t.numel(), generator=g).reshape(sh).to(dt) if dt != torch.bfloat16 else t
            run(f"max_dim/{dt}/{sh}/{dim}", lambda x, dim=dim: torch.max(x, dim), [tt], dt)
            run(f"argmax/{dt}/{sh}/{dim}", lambda x, dim=dim: torch.argmax(x, dim), [tt], dt)
            run(f"argmin/{dt}/{sh}/{dim}", lambda x, dim=dim: torch.argmin(x, dim, keepdim=True), [tt], dt)
            run(f"cumsum/{dt}/{sh}/{dim}", lambda x, dim=dim: torch.cumsum(x, dim), [t if dt != torch.bfloat16 else t.float()], torch.float32 if dt == torch.bfloat16 else dt)
for sh in [(3, 5), (2, 3, 4)]:
    b = rnd(sh, torch.bool)
    run(f"any/{sh}", torch.any, [b], torch.bool); run(f"all/{sh}", torch.all, [b], torch.bool)
    run(f"any_dim/{sh}", lambda x: torch.any(x, 1), [b], torch.bool); run(f"all_dim/{sh}", lambda x: torch.all(x, -1), [b], torch.bool)
# ---- softmax family
for dt in [torch.float32, torch.bfloat16, torch.float16]:
    for sh, dims in [((7, 1031), [0, 1]), ((3, 5, 7), [0, 1, 2]), ((2, 12, 16, 16), [-1]), ((4, 30522), [1]), ((1, 1), [0])]:
        for dim in dims:
            run(f"softmax/{dt}/{sh}/{dim}", lambda x, dim=dim: F.softmax(x, dim), [rnd(sh, dt)], dt, grad=dt != torch.float16)
            run(f"log_softmax/{dt}/{sh}/{dim}", lambda x, dim=dim: F.log_softmax(x, dim), [rnd(sh, dt)], dt, grad=dt != torch.float16)
# ---- shape ops
run("cat", lambda a, b: torch.cat([a, b], 1), [rnd((3, 5), torch.float32), rnd((3, 2), torch.float32)], torch.float32)
run("cat_cl", lambda a, b: torch.cat([a, b], 1), [rnd((2, 8, 4, 4), torch.bfloat16).contiguous(memory_format=torch.channels_last), rnd((2, 16, 4, 4), torch.bfloat16).contiguous(memory_format=torch.channels_last)], torch.bfloat16)
run("cat0", lambda a, b: torch.cat([a, b], 0), [rnd((3, 5), torch.int64), rnd((0, 5), torch.int64)], torch.int64)
run("stack", lambda a, b: torch.stack([a, b], -1), [rnd((3, 5), torch.float16), rnd((3, 5), torch.float16)], torch.float16)
run("permute_contig", lambda a: a.permute(0, 2, 3, 1).contiguous(), [rnd((2, 3, 4, 5), torch.float32)], torch.float32)
run("transpose_contig_big", lambda a: a.t().contiguous(), [rnd((1031, 257), torch.bfloat16)], torch.bfloat16)
for src, dst in itertools.product([torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.int32, torch.uint8, torch.bool, torch.float64], repeat=2):
    t = rnd((5, 7), src)
    if src == torch.uint8 or dst == torch.uint8: t = t.abs() if src != torch.bool else t
    run(f"cast/{src}/{dst}", lambda x, dst=dst: x.to(dst), [t], torch.float32)
run("expand_contig", lambda a: a.expand(4, 3, 5).contiguous(), [rnd((3, 1), torch.float32)], torch.float32)
run("flip", lambda a: a.flip(1), [rnd((3, 5), torch.float32)], torch.float32)
run("roll", lambda a: a.roll(2, 1), [rnd((3, 5), torch.float32)], torch.float32)
run("repeat", lambda a: a.repeat(2, 3), [rnd((3, 5), torch.float32)], torch.float32)
run("tril", lambda a: a.tril(-1), [rnd((6, 5), torch.float32)], torch.float32)
run("triu", lambda a: a.triu(1), [rnd((2, 6, 5), torch.bfloat16)], torch.bfloat16)
run("arange", lambda a: torch.arange(0, 37, 3, device=a.device), [rnd((1,), torch.float32)], torch.int64)
run("linspace", lambda a: torch.linspace(0, 1, 13, device=a.device), [rnd((1,), torch.float32)], torch.float32)
run("fill", lambda a: a.clone().fill_(3.5), [rnd((3, 5), torch.bfloat16)], torch.bfloat16)
run("zero_strided", lambda a: a.clone()[:, ::2].zero_(), [rnd((3, 6), torch.float32)], torch.float32)
run("clone_cl", lambda a: a.clone(memory_format=torch.channels_last), [rnd((2, 3, 4, 5), torch.float32)], torch.float32)
# ---- indexing
idx = torch.randint(0, 7, (11,), generator=g)
for dt in [torch.float32, torch.bfloat16, torch.int64]:
    src = rnd((7, 9), dt)
    run(f"index_select0/{dt}", lambda x, i: x.index_select(0, i), [src, idx], dt)
    run(f"index_select1/{dt}", lambda x, i: x.index_select(1, i), [src, idx], dt)
    run(f"gather/{dt}", lambda x, i: x.gather(1, i), [src, torch.randint(0, 9, (7, 4), generator=g)], dt)
    run(f"adv_index/{dt}", lambda x, i, j: x[i, j], [src, idx, torch.randint(0, 9, (11,), generator=g)], dt)
    run(f"bool_index/{dt}", lambda x, m: x[m], [src, rnd((7, 9), torch.bool)], dt)
    run(f"masked_fill/{dt}", lambda x, m: x.masked_fill(m, 2), [src, rnd((7, 9), torch.bool)], dt)
    run(f"index_put/{dt}", lambda x, i, v: x.clone().index_put_((i,), v, accumulate=False), [src, torch.tensor([0, 3, 5]), rnd((3, 9), dt)], dt)
    if dt != torch.int64:
        run(f"index_put_acc/{dt}", lambda x, i, v: x.clone().index_put_((i,), v, accumulate=True), [src.float(), torch.tensor([0, 3, 3, 5]), rnd((4, 9), torch.float32)], torch.float32)
        run(f"scatter_add/{dt}", lambda x, i, v: x.clone().scatter_add_(1, i, v), [src.float(), torch.randint(0, 9, (7, 4), generator=g), rnd((7, 4), torch.float32)], torch.float32)
    run(f"nonzero/{dt}", torch.nonzero, [rnd((7, 9), dt)], dt)
    for k, largest in [(1, True), (4, False), (9, True)]:
        vals = torch.randperm(63, generator=g).reshape(7, 9).to(dt)
        run(f"topk/{dt}/{k}/{largest}", lambda x, k=k, l=largest: torch.topk(x, k, largest=l), [vals], dt)
    vals = torch.randperm(63, generator=g).reshape(7, 9).to(dt)
    run(f"sort/{dt}", lambda x: torch.sort(x, 1, descending=True), [vals], dt)
    run(f"sort0/{dt}", lambda x: torch.sort(x, 0), [vals], dt)
run("sort_long", lambda x: torch.sort(x), [torch.randperm(100003, generator=g).float()], torch.float32)
run("unique", lambda x: torch.unique(x, return_inverse=True, return_counts=True), [torch.randint(0, 20, (200,), generator=g)], torch.int64)
emb = rnd((50, 24), torch.float32)
run("embedding", lambda w, i: F.embedding(i, w, padding_idx=3), [emb, torch.randint(0, 50, (4, 9), generator=g)], torch.float32, grad=True)
run("embedding_bf16", lambda w, i: F.embedding(i, w), [emb.bfloat16(), torch.randint(0, 50, (4, 9), generator=g)], torch.bfloat16, grad=True)
run("masked_select", torch.masked_select, [rnd((7, 9), torch.float32), rnd((7, 9), torch.bool)], torch.float32)
run("one_hot", lambda i: F.one_hot(i, 12), [torch.randint(0, 12, (5, 3), generator=g)], torch.int64)
# ---- pooling
for dt in [torch.float32, torch.bfloat16]:
    for sh in [(2, 8, 13, 13), (1, 3, 7, 9), (2, 16, 8, 8)]:
        for ln, t in layouts(sh, dt):
            if ln not in ("c", "cl"): continue
            # distinct values so that ties do not decide the gradient
            t = (torch.randperm(t.numel(), generator=g).reshape(sh).float() / t.numel()).to(dt)
            if ln == "cl": t = t.contiguous(memory_format=torch.channels_last)
            run(f"maxpool/{dt}/{sh}/{ln}", lambda x: F.max_pool2d(x, 3, 2, 1), [t], dt, grad=dt == torch.float32)
            run(f"maxpool_ceil/{dt}/{sh}/{ln}", lambda x: F.max_pool2d(x, 2, 2, 0, ceil_mode=True), [t], dt, grad=dt == torch.float32)
            run(f"avgpool/{dt}/{sh}/{ln}", lambda x: F.avg_pool2d(x, 3, 2, 1), [t], dt, grad=True)
            run(f"avgpool_nopad/{dt}/{sh}/{ln}", lambda x: F.avg_pool2d(x, 3, 1, 1, count_include_pad=False), [t], dt, grad=True)
            run(f"adaptive_avg1/{dt}/{sh}/{ln}", lambda x: F.adaptive_avg_pool2d(x, 1), [t], dt, grad=True)
            run(f"adaptive_avg3/{dt}/{sh}/{ln}", lambda x: F.adaptive_avg_pool2d(x, (3, 2)), [t], dt, grad=True)
            run(f"adaptive_max/{dt}/{sh}/{ln}", lambda x: F.adaptive_max_pool2d(x, (3, 2)), [t], dt, grad=dt == torch.float32)
            run(f"up_nearest/{dt}/{sh}/{ln}", lambda x: F.interpolate(x, scale_factor=2, mode="nearest"), [t], dt, grad=True)
            run(f"up_bilinear/{dt}/{sh}/{ln}", lambda x: F.interpolate(x, size=(9, 11), mode="bilinear", align_corners=False), [t], dt, grad=True)
            run(f"up_bilinear_ac/{dt}/{sh}/{ln}", lambda x: F.interpolate(x, scale_factor=2, mode="bilinear", align_corners=True), [t], dt, grad=True)
# ---- norms
for dt in [torch.float32, torch.bfloat16]:
    for C, cl in [(3, False), (5, True), (8, True), (64, True), (24, False)]:
        x = rnd((4, C, 6, 6), dt)
        if cl: x = x.contiguous(memory_format=torch.channels_last)
        w, b = rnd((C,), torch.float32), rnd((C,), torch.float32)
        run(f"bn_train/{dt}/{C}/{cl}", lambda x, w, b: F.batch_norm(x, None, None, w.to(x.dtype) if False else w, b, True, 0.1, 1e-5), [x, w, b], dt, grad=True)
        rm, rv = rnd((C,), torch.float32), rnd((C,), torch.float32, True)
        run(f"bn_eval/{dt}/{C}/{cl}", lambda x, w, b, rm=rm, rv=rv: F.batch_norm(x, rm.to(x.device), rv.to(x.device), w, b, False, 0.1, 1e-5), [x, w, b], dt, grad=True)
    for cols in [13, 768, 1000, 4096]:
        x = rnd((9, cols), dt)
        w, b = rnd((cols,), dt), rnd((cols,), dt)
        run(f"layer_norm/{dt}/{cols}", lambda x, w, b, cols=cols: F.layer_norm(x, (cols,), w, b), [x, w, b], dt, grad=True)
    run(f"layer_norm_noaffine/{dt}", lambda x: F.layer_norm(x, (5, 7)), [rnd((3, 5, 7), dt)], dt, grad=True)
    run(f"group_norm/{dt}", lambda x, w, b: F.group_norm(x, 4, w, b), [rnd((2, 8, 5, 5), dt), rnd((8,), dt), rnd((8,), dt)], dt, grad=True)
# ---- matmul family
for dt in FDT:
    for m, k, n in [(7, 13, 5), (1, 1, 1), (128, 64, 256), (33, 200, 65), (5, 0, 3), (257, 129, 8)]:
        a, b = rnd((m, k), dt), rnd((k, n), dt)
        run(f"mm/{dt}/{m}x{k}x{n}", torch.mm, [a, b], dt, grad=dt != torch.float16)
        run(f"mm_tn/{dt}/{m}x{k}x{n}", lambda a, b: a.t() @ b.t(), [rnd((k, m), dt), rnd((n, k), dt)], dt)
        run(f"addmm/{dt}/{m}x{k}x{n}", lambda c, a, b: torch.addmm(c, a, b, beta=0.5, alpha=2.0), [rnd((n,), dt), a, b], dt)
        if k: run(f"linear/{dt}/{m}x{k}x{n}", F.linear, [rnd((3, m, k), dt), rnd((n, k), dt), rnd((n,), dt)], dt, grad=dt != torch.float16)
    run(f"bmm/{dt}", torch.bmm, [rnd((4, 7, 13), dt), rnd((4, 13, 5), dt)], dt, grad=dt != torch.float16)
    run(f"baddbmm/{dt}", lambda c, a, b: torch.baddbmm(c, a, b, beta=0.3, alpha=1.5), [rnd((4, 7, 5), dt), rnd((4, 7, 13), dt), rnd((4, 13, 5), dt)], dt)
    run(f"matmul_bcast/{dt}", torch.matmul, [rnd((2, 3, 7, 13), dt), rnd((13, 5), dt)], dt)
    run(f"matmul_vec/{dt}", torch.matmul, [rnd((7, 13), dt), rnd((13,), dt)], dt)
    run(f"dot/{dt}", torch.dot, [rnd((13,), dt), rnd((13,), dt)], dt)
# ---- convolution
CONV = [(3, 16, 3, 1, 1, 1, 1), (8, 16, 3, 2, 1, 1, 1), (16, 32, 1, 1, 0, 1, 1), (16, 16, 3, 1, 2, 2, 1), (16, 32, 3, 1, 1, 1, 4), (16, 16, 3, 1, 1, 1, 16),
        (5, 7, 3, 1, 1, 1, 1), (64, 64, 3, 1, 1, 1, 1), (8, 8, 5, 2, 2, 1, 1), (24, 40, (1, 3), 1, (0, 1), 1, 1)]
for dt in [torch.float32, torch.bfloat16]:
    for cin, cout, k, s, p, d, gr in CONV:
        ks = (k, k) if isinstance(k, int) else k
        x = rnd((2, cin, 9, 11), dt)
        w = (rnd((cout, cin // gr) + ks, dt).float() * 0.2).to(dt)
        bias = rnd((cout,), dt)
        for cl in (False, True):
            xx = x.contiguous(memory_format=torch.channels_last) if cl else x
            run(f"conv2d/{dt}/{cin}-{cout}-{k}-{s}-{p}-{d}-{gr}/{cl}", lambda x, w, b, s=s, p=p, d=d, gr=gr: F.conv2d(x, w, b, s, p, d, gr), [xx, w, bias], dt, grad=True)
    run(f"conv_transpose/{dt}", lambda x, w: F.conv_transpose2d(x, w, None, 2, 1, 1), [rnd((2, 16, 5, 5), dt), (rnd((16, 8, 3, 3), dt).float() * 0.2).to(dt)], dt, grad=True)
    run(f"conv1d/{dt}", lambda x, w: F.conv1d(x, w, None, 1, 1), [rnd((2, 8, 20), dt), (rnd((16, 8, 3), dt).float() * 0.2).to(dt)], dt, grad=True)
# ---- losses
for dt in [torch.float32, torch.bfloat16]:
    lg = rnd((9, 11), dt); tg = torch.randint(0, 11, (9,), generator=g); tg[2] = -100
    wt = rnd((11,), torch.float32, True).to(dt)
    for red in ("mean", "sum", "none"):
        run(f"ce/{dt}/{red}", lambda x, t, red=red: F.cross_entropy(x, t, reduction=red), [lg, tg], dt, grad=True)
        run(f"ce_w/{dt}/{red}", lambda x, t, red=red, wt=wt: F.cross_entropy(x, t, wt.to(x.device), reduction=red), [lg, tg], dt, grad=True)
        run(f"ce_ls/{dt}/{red}", lambda x, t, red=red: F.cross_entropy(x, t, reduction=red, label_smoothing=0.1), [lg, tg], dt, grad=True)
        run(f"nll/{dt}/{red}", lambda x, t, red=red: F.nll_loss(F.log_softmax(x, 1), t, reduction=red), [lg, tg], dt, grad=True)
        run(f"mse/{dt}/{red}", lambda x, y, red=red: F.mse_loss(x, y, reduction=red), [lg, rnd((9, 11), dt)], dt, grad=True)
        run(f"smooth_l1/{dt}/{red}", lambda x, y, red=red: F.smooth_l1_loss(x, y, reduction=red, beta=0.5), [lg, rnd((9, 11), dt)], dt, grad=True)
        run(f"l1/{dt}/{red}", lambda x, y, red=red: F.l1_loss(x, y, reduction=red), [lg, rnd((9, 11), dt)], dt, grad=True)
        run(f"bce_logits/{dt}/{red}", lambda x, y, red=red: F.binary_cross_entropy_with_logits(x, y, reduction=red), [lg, torch.rand((9, 11), generator=g).to(dt)], dt, grad=True)
        run(f"bce/{dt}/{red}", lambda x, y, red=red: F.binary_cross_entropy(torch.sigmoid(x), y, reduction=red), [lg, torch.rand((9, 11), generator=g).to(dt)], dt, grad=True)
    run(f"nll2d/{dt}", lambda x, t: F.cross_entropy(x, t), [rnd((2, 5, 4, 4), dt), torch.randint(0, 5, (2, 4, 4), generator=g)], dt, grad=True)
    run(f"dropout_eval/{dt}", lambda x: F.dropout(x, 0.5, False), [lg], dt)
    run(f"dropout_p0/{dt}", lambda x: F.dropout(x, 0.0, True), [lg], dt)
    run(f"kl_div/{dt}", lambda x, y: F.kl_div(F.log_softmax(x, 1), F.softmax(y, 1), reduction="batchmean"), [lg, rnd((9, 11), dt)], dt, grad=True)

torch.b200.synchronize()
print(f"ok {n_ok} fail {len(fails)}")
_log.write(f"TOTAL ok {n_ok} fail {len(fails)}\n")
if not torch.b200.is_hostsim():
    _log.write(f"flag {catch_b200.ops.capi.read_error_flag()}\n")
_log.close()
