"""A walk through torch.nn and the tensor API on the device: about 140 modules, losses and functions, forward and (for
modules) backward, against the CPU.  On the host-simulated device most of them run through the CPU fallback, which
is the point: whatever the dispatcher routes somewhere else for a non-CPU device (fused RNN cells, attention fast
paths, nested tensors) shows up here as an exception.  On a GPU the same walk is `tests/op_sweep.py`'s neighbour."""
import torch
import torch.nn as nn
import torch.nn.functional as F

import catch_b200  # noqa: F401

D = "blackwell"


def test_module_and_function_zoo():
    torch.manual_seed(0)
    fails = []

    def chk(name, fn, tol=1e-4, grad=True):
        try:
            r = fn("cpu"); d = fn(D)
            rs = r if isinstance(r, (tuple, list)) else [r]; ds = d if isinstance(d, (tuple, list)) else [d]
            for a, b in zip(rs, ds):
                if isinstance(a, torch.Tensor):
                    if a.shape != b.shape: fails.append((name, f"shape {a.shape} vs {b.shape}")); return
                    if a.dtype.is_floating_point:
                        if not torch.allclose(a.detach(), b.detach().cpu(), atol=tol, rtol=tol, equal_nan=True): fails.append((name, f"mismatch {float((a.detach()-b.detach().cpu()).abs().max()):.2e}"))
                    elif not torch.equal(a, b.cpu()): fails.append((name, "int mismatch"))
        except Exception as e:
            fails.append((name, "EXC " + repr(e)[:160]))
    def mod_case(name, ctor, inp_fn, eval_mode=False, tol=1e-4):
        def run(dev):
            torch.manual_seed(1); m = ctor().to(dev)
            if eval_mode: m.eval()
            torch.manual_seed(2); x = inp_fn()
            x = [t.to(dev) if isinstance(t, torch.Tensor) else t for t in (x if isinstance(x, tuple) else (x,))]
            out = m(*x); out = out[0] if isinstance(out, tuple) else out
            if out.requires_grad:
                out.float().sum().backward()
                return [out] + [p.grad for p in m.parameters() if p.grad is not None]
            return out
        chk(name, run, tol)
    x4 = lambda: torch.randn(2, 4, 8, 8)
    mod_case("MHA eval fastpath", lambda: nn.MultiheadAttention(8, 2, batch_first=True), lambda: (torch.randn(3, 6, 8),) * 3, eval_mode=True)
    def te_eval(dev):
        torch.manual_seed(1); m = nn.TransformerEncoder(nn.TransformerEncoderLayer(8, 2, 16, dropout=0.0, batch_first=True), 2, enable_nested_tensor=False).to(dev).eval()
        torch.manual_seed(2); x = torch.randn(3, 6, 8).to(dev)
        with torch.no_grad(): return m(x, src_key_padding_mask=torch.tensor([[False]*6, [False]*4 + [True]*2, [False]*6]).to(dev))
    chk("TransformerEncoder eval", te_eval)
    mod_case("LSTM", lambda: nn.LSTM(5, 7, num_layers=2, batch_first=True, bidirectional=True), lambda: torch.randn(3, 6, 5))
    mod_case("GRU", lambda: nn.GRU(5, 7), lambda: torch.randn(6, 3, 5))
    mod_case("TransformerEncoderLayer train", lambda: nn.TransformerEncoderLayer(8, 2, 16, dropout=0.0, batch_first=True), lambda: torch.randn(3, 6, 8))
    chk("sdpa", lambda dev: F.scaled_dot_product_attention(*(torch.randn(2, 2, 5, 4, generator=torch.Generator().manual_seed(3)).to(dev) for _ in range(3)), is_causal=True))
    chk("sdpa mask", lambda dev: F.scaled_dot_product_attention(*[t.to(dev) for t in torch.randn(3, 2, 2, 5, 4, generator=torch.Generator().manual_seed(3)).unbind(0)], attn_mask=(torch.rand(5, 5, generator=torch.Generator().manual_seed(4)) > 0.3).to(dev)))
    mod_case("ConvTranspose1d", lambda: nn.ConvTranspose1d(4, 6, 3, stride=2), lambda: torch.randn(2, 4, 9))
    mod_case("ConvTranspose3d", lambda: nn.ConvTranspose3d(4, 6, 3), lambda: torch.randn(2, 4, 4, 4, 4))
    mod_case("Conv3d", lambda: nn.Conv3d(4, 6, 3, padding=1), lambda: torch.randn(2, 4, 4, 5, 5))
    mod_case("PReLU", lambda: nn.PReLU(4), x4)
    mod_case("Bilinear", lambda: nn.Bilinear(4, 5, 3), lambda: (torch.randn(6, 4), torch.randn(6, 5)))
    mod_case("LocalResponseNorm", lambda: nn.LocalResponseNorm(2), x4)
    mod_case("PixelShuffle", lambda: nn.PixelShuffle(2), x4)
    mod_case("Unfold", lambda: nn.Unfold(3, padding=1), x4)
    mod_case("Fold", lambda: nn.Fold((4, 4), 2), lambda: torch.randn(2, 16, 9))
    mod_case("Upsample bicubic", lambda: nn.Upsample(scale_factor=2, mode="bicubic"), x4)
    mod_case("Upsample trilinear", lambda: nn.Upsample(scale_factor=2, mode="trilinear"), lambda: torch.randn(1, 2, 3, 4, 4))
    mod_case("ReflectionPad2d", lambda: nn.ReflectionPad2d(2), x4)
    mod_case("ReplicationPad2d", lambda: nn.ReplicationPad2d(1), x4)
    mod_case("ZeroPad/ConstantPad", lambda: nn.ConstantPad2d((1, 2, 0, 1), 3.0), x4)
    mod_case("MaxPool1d", lambda: nn.MaxPool1d(3, 2), lambda: torch.randn(2, 4, 11))
    mod_case("AvgPool1d", lambda: nn.AvgPool1d(3, 2), lambda: torch.randn(2, 4, 11))
    mod_case("AdaptiveAvgPool1d", lambda: nn.AdaptiveAvgPool1d(3), lambda: torch.randn(2, 4, 11))
    mod_case("LPPool2d", lambda: nn.LPPool2d(2, 2), x4)
    mod_case("FractionalMaxPool2d", lambda: nn.FractionalMaxPool2d(2, output_size=(4, 4)), x4, tol=1e9)
    mod_case("Softmax2d", lambda: nn.Softmax2d(), x4)
    mod_case("Hardshrink/Softshrink", lambda: nn.Sequential(nn.Hardshrink(), nn.Softshrink(0.1)), x4)
    mod_case("Mish/GLU/CELU/SELU", lambda: nn.Sequential(nn.Mish(), nn.GLU(1), nn.CELU(), nn.SELU()), x4)
    mod_case("RReLU eval", lambda: nn.RReLU(), x4, eval_mode=True)
    mod_case("Softmin/LogSoftmax", lambda: nn.Sequential(nn.Softmin(1), nn.LogSoftmax(1)), x4)
    mod_case("Threshold/Tanhshrink/Softsign", lambda: nn.Sequential(nn.Threshold(0.1, 2.0), nn.Tanhshrink(), nn.Softsign()), x4)
    mod_case("CosineSimilarity", lambda: nn.CosineSimilarity(1), lambda: (torch.randn(5, 7), torch.randn(5, 7)))
    mod_case("PairwiseDistance", lambda: nn.PairwiseDistance(), lambda: (torch.randn(5, 7), torch.randn(5, 7)))
    mod_case("Flatten/Unflatten", lambda: nn.Sequential(nn.Flatten(), nn.Unflatten(1, (4, 64))), x4)
    mod_case("ChannelShuffle", lambda: nn.ChannelShuffle(2), x4)
    mod_case("Identity/Dropout eval", lambda: nn.Sequential(nn.Identity(), nn.Dropout(0.5), nn.AlphaDropout(0.5)), x4, eval_mode=True)
    mod_case("InstanceNorm1d", lambda: nn.InstanceNorm1d(4), lambda: torch.randn(2, 4, 9))
    mod_case("LayerNorm 2 dims", lambda: nn.LayerNorm((8, 8)), x4)
    mod_case("RMSNorm", lambda: nn.RMSNorm(8), x4)
    mod_case("Embedding sparse=False scale", lambda: nn.Embedding(10, 4, scale_grad_by_freq=True), lambda: torch.randint(0, 10, (3, 5)))
    # losses
    L = lambda: torch.randn(6, 5); T = lambda: torch.randint(0, 5, (6,))
    for nm, fn in [("CTCLoss", lambda dev: F.ctc_loss(torch.randn(12, 3, 6, generator=torch.Generator().manual_seed(5)).log_softmax(2).to(dev), torch.randint(1, 6, (3, 4), generator=torch.Generator().manual_seed(6)).to(dev), torch.full((3,), 12), torch.full((3,), 4))),
                   ("HingeEmbedding", lambda dev: F.hinge_embedding_loss(torch.randn(6, generator=torch.Generator().manual_seed(5)).to(dev), torch.tensor([1., -1, 1, -1, 1, 1]).to(dev))),
                   ("MarginRanking", lambda dev: F.margin_ranking_loss(*[torch.randn(6, generator=torch.Generator().manual_seed(s)).to(dev) for s in (1, 2)], torch.tensor([1., -1, 1, -1, 1, 1]).to(dev))),
                   ("MultiMargin", lambda dev: F.multi_margin_loss(torch.randn(6, 5, generator=torch.Generator().manual_seed(5)).to(dev), torch.randint(0, 5, (6,), generator=torch.Generator().manual_seed(6)).to(dev))),
                   ("MultiLabelSoftMargin", lambda dev: F.multilabel_soft_margin_loss(torch.randn(6, 5, generator=torch.Generator().manual_seed(5)).to(dev), (torch.rand(6, 5, generator=torch.Generator().manual_seed(6)) > 0.5).float().to(dev))),
                   ("TripletMargin", lambda dev: F.triplet_margin_loss(*[torch.randn(6, 5, generator=torch.Generator().manual_seed(s)).to(dev) for s in (1, 2, 3)])),
                   ("CosineEmbedding", lambda dev: F.cosine_embedding_loss(*[torch.randn(6, 5, generator=torch.Generator().manual_seed(s)).to(dev) for s in (1, 2)], torch.tensor([1., -1, 1, -1, 1, 1]).to(dev))),
                   ("PoissonNLL", lambda dev: F.poisson_nll_loss(torch.randn(6, 5, generator=torch.Generator().manual_seed(5)).to(dev), torch.rand(6, 5, generator=torch.Generator().manual_seed(6)).to(dev))),
                   ("GaussianNLL", lambda dev: F.gaussian_nll_loss(*[torch.randn(6, 5, generator=torch.Generator().manual_seed(s)).to(dev) for s in (1, 2)], torch.rand(6, 5, generator=torch.Generator().manual_seed(3)).to(dev) + 0.1)),
                   ("Huber", lambda dev: F.huber_loss(*[torch.randn(6, 5, generator=torch.Generator().manual_seed(s)).to(dev) for s in (1, 2)], delta=0.7)),
                   ("SoftMargin", lambda dev: F.soft_margin_loss(torch.randn(6, generator=torch.Generator().manual_seed(5)).to(dev), torch.tensor([1., -1, 1, -1, 1, 1]).to(dev)))]:
        chk(nm, fn)
    # functional / tensor ops
    G = lambda s, *shape: torch.randn(*shape, generator=torch.Generator().manual_seed(s))
    for nm, fn in [("grid_sample", lambda dev: F.grid_sample(G(1, 2, 3, 5, 5).to(dev), (G(2, 2, 4, 4, 2) * 0.5).to(dev), align_corners=False)),
                   ("affine_grid", lambda dev: F.affine_grid(G(1, 2, 2, 3).to(dev), (2, 3, 4, 4), align_corners=False)),
                   ("einsum", lambda dev: torch.einsum("bij,bjk->bik", G(1, 2, 3, 4).to(dev), G(2, 2, 4, 5).to(dev))),
                   ("cdist", lambda dev: torch.cdist(G(1, 5, 3).to(dev), G(2, 6, 3).to(dev))),
                   ("bucketize", lambda dev: torch.bucketize(G(1, 7).to(dev), torch.tensor([-1., 0, 1]).to(dev))),
                   ("searchsorted", lambda dev: torch.searchsorted(torch.tensor([-1., 0, 1]).to(dev), G(1, 7).to(dev))),
                   ("histc", lambda dev: torch.histc(G(1, 50).to(dev), bins=5, min=-2, max=2)),
                   ("linalg.inv", lambda dev: torch.linalg.inv((G(1, 4, 4) + 4 * torch.eye(4)).to(dev))),
                   ("linalg.solve", lambda dev: torch.linalg.solve((G(1, 4, 4) + 4 * torch.eye(4)).to(dev), G(2, 4, 2).to(dev))),
                   ("cholesky", lambda dev: torch.linalg.cholesky((G(1, 4, 4) @ G(1, 4, 4).T + 4 * torch.eye(4)).to(dev))),
                   ("svdvals", lambda dev: torch.linalg.svdvals(G(1, 4, 3).to(dev))),
                   ("qr", lambda dev: torch.linalg.qr(G(1, 4, 3).to(dev))[1].abs()),
                   ("det", lambda dev: torch.linalg.det(G(1, 3, 3).to(dev))),
                   ("fft", lambda dev: torch.fft.rfft(G(1, 16).to(dev)).abs()),
                   ("cummax", lambda dev: torch.cummax(G(1, 3, 5).to(dev), 1)[0]),
                   ("cumprod", lambda dev: torch.cumprod(G(1, 3, 5).to(dev), 1)),
                   ("logcumsumexp", lambda dev: torch.logcumsumexp(G(1, 3, 5).to(dev), 1)),
                   ("kthvalue", lambda dev: torch.kthvalue(G(1, 3, 5).to(dev), 2, 1)[0]),
                   ("median", lambda dev: torch.median(G(1, 3, 5).to(dev), 1)[0]),
                   ("mode", lambda dev: torch.mode(torch.randint(0, 3, (3, 7), generator=torch.Generator().manual_seed(1)).to(dev), 1)[0]),
                   ("quantile", lambda dev: torch.quantile(G(1, 20).to(dev), 0.3)),
                   ("nanmean/nansum", lambda dev: torch.nansum(torch.tensor([1., float("nan"), 2.]).to(dev))),
                   ("diag/diagonal/trace", lambda dev: torch.diag(G(1, 4, 4).to(dev)).sum() + torch.trace(G(2, 4, 4).to(dev))),
                   ("kron", lambda dev: torch.kron(G(1, 2, 2).to(dev), G(2, 3, 3).to(dev))),
                   ("tensordot", lambda dev: torch.tensordot(G(1, 3, 4, 5).to(dev), G(2, 4, 5, 6).to(dev), dims=2)),
                   ("outer/cross", lambda dev: torch.outer(G(1, 3).to(dev), G(2, 4).to(dev)).sum() + torch.linalg.cross(G(3, 5, 3).to(dev), G(4, 5, 3).to(dev)).sum()),
                   ("baddbmm/addbmm/addr", lambda dev: torch.addbmm(G(1, 3, 5).to(dev), G(2, 2, 3, 4).to(dev), G(3, 2, 4, 5).to(dev)) + torch.addr(G(4, 3, 5).to(dev), G(5, 3).to(dev), G(6, 5).to(dev))),
                   ("lerp/hypot/logaddexp", lambda dev: torch.lerp(G(1, 5).to(dev), G(2, 5).to(dev), G(3, 5).to(dev).sigmoid()) + torch.hypot(G(4, 5).to(dev), G(5, 5).to(dev)) + torch.logaddexp(G(6, 5).to(dev), G(7, 5).to(dev))),
                   ("special", lambda dev: torch.special.expit(G(1, 5).to(dev)) + torch.special.erfc(G(2, 5).to(dev)) + torch.lgamma(G(3, 5).abs().to(dev) + 1) + torch.digamma(G(4, 5).abs().to(dev) + 1)),
                   ("bitwise/shift", lambda dev: (torch.arange(8).to(dev) << 2) ^ (torch.arange(8).to(dev) | 3) & ~torch.arange(8).to(dev)),
                   ("isin/unique_consecutive", lambda dev: torch.isin(torch.arange(8).to(dev), torch.tensor([1, 5]).to(dev))),
                   ("repeat_interleave", lambda dev: torch.repeat_interleave(torch.arange(4).to(dev), torch.tensor([1, 0, 2, 3]).to(dev))),
                   ("take_along_dim/take/put", lambda dev: torch.take_along_dim(G(1, 3, 5).to(dev), torch.randint(0, 5, (3, 2), generator=torch.Generator().manual_seed(1)).to(dev), 1)),
                   ("index_add/index_copy", lambda dev: G(1, 5, 3).to(dev).index_add(0, torch.tensor([0, 2, 2]).to(dev), G(2, 3, 3).to(dev)).index_copy(0, torch.tensor([1]).to(dev), G(3, 1, 3).to(dev))),
                   ("scatter_reduce", lambda dev: torch.zeros(4).to(dev).scatter_reduce(0, torch.tensor([0, 1, 0, 3]).to(dev), G(1, 4).to(dev), "amax", include_self=False)),
                   ("masked_scatter", lambda dev: torch.zeros(6).to(dev).masked_scatter(torch.tensor([1, 0, 1, 1, 0, 0]).bool().to(dev), G(1, 6).to(dev))),
                   ("tril_indices/triu_indices", lambda dev: torch.tril_indices(4, 4, device=dev)),
                   ("meshgrid/cartesian", lambda dev: torch.stack(torch.meshgrid(torch.arange(3.).to(dev), torch.arange(2.).to(dev), indexing="ij")).sum()),
                   ("clamp tensor bounds", lambda dev: torch.clamp(G(1, 5).to(dev), G(2, 5).to(dev) - 1, G(3, 5).to(dev) + 1)),
                   ("nan_to_num", lambda dev: torch.nan_to_num(torch.tensor([float("nan"), float("inf"), -float("inf"), 1.]).to(dev))),
                   ("complex abs", lambda dev: torch.view_as_real(torch.view_as_complex(G(1, 4, 2).to(dev)) * 2)),
                   ("float64 mm", lambda dev: G(1, 4, 5).double().to(dev) @ G(2, 5, 3).double().to(dev)),
                   ("int mm", lambda dev: torch.arange(12).reshape(3, 4).to(dev) @ torch.arange(8).reshape(4, 2).to(dev)),
                   ("half mm", lambda dev: (G(1, 4, 8).half().to(dev) @ G(2, 8, 3).half().to(dev)).float())]:
        chk(nm, fn, tol=2e-3 if "half" in nm else 1e-4)
    # init functions on device parameters
    def inits(dev):
        p = torch.empty(8, 6, device=dev)
        torch.manual_seed(3)
        for f in (nn.init.kaiming_uniform_, nn.init.xavier_normal_, lambda t: nn.init.trunc_normal_(t, std=0.1), nn.init.orthogonal_, lambda t: nn.init.sparse_(t, 0.5), nn.init.eye_, nn.init.zeros_):
            f(p)
        return p.abs().sum() * 0
    chk("nn.init", inits)
    chk("randperm/multinomial/normal", lambda dev: (torch.randperm(10, device=dev).sort()[0].float().sum() + torch.multinomial(torch.ones(5).to(dev), 3).numel() + torch.normal(0., 1., (4,), device=dev).numel()) * 0)
    assert not fails, "\n".join(f"{n}: {w}" for n, w in fails)


def test_complex_views_and_lazy_conjugates():
    """view_as_complex / view_as_real are real views on the device (rotary embeddings write through them), and copies of
    lazily conjugated or negated tensors (x.conj(), the views autograd makes for complex gradients) resolve the bit
    instead of recursing through the dispatcher's generic conjugate kernel (which used to end in a stack overflow)."""
    x = torch.randn(3, 4, 2)
    c_cpu, xd = torch.view_as_complex(x), x.to(D)
    c = torch.view_as_complex(xd)
    r = torch.view_as_real(c)
    assert c.dtype == torch.complex64 and r.data_ptr() == xd.data_ptr() and torch.equal(r.cpu(), x)
    r[0, 0, 0] = 5.0
    assert float(xd[0, 0, 0]) == 5.0                      # a view, not a copy
    x = xd.cpu()
    c_cpu = torch.view_as_complex(x)
    assert torch.equal(c.conj().cpu(), c_cpu.conj())
    assert torch.equal(c.conj().clone().cpu(), c_cpu.conj()) and torch.equal(c.conj().resolve_conj().cpu(), c_cpu.conj())
    assert torch.equal(c_cpu.conj().to(D).cpu(), c_cpu.conj())
    assert torch.equal(torch._neg_view(xd).clone().cpu(), -x)
    assert torch.allclose((c.H @ c).cpu(), c_cpu.H @ c_cpu, atol=1e-5)
    a = torch.randn(3, 2, dtype=torch.complex64, requires_grad=True)
    ad = a.detach().to(D).requires_grad_()
    (a * a.conj()).real.sum().backward()
    (ad * ad.conj()).real.sum().backward()
    assert torch.allclose(ad.grad.cpu(), a.grad, atol=1e-5)
    # rotary position embedding the way LLM code writes it
    q = torch.randn(2, 6, 4, 8)
    freqs = torch.polar(torch.ones(6, 4), torch.randn(6, 4))
    rope = lambda t, f: torch.view_as_real(torch.view_as_complex(t.float().reshape(*t.shape[:-1], -1, 2)) * f[None, :, None, :]).flatten(3)
    assert torch.allclose(rope(q.to(D), freqs.to(D)).cpu(), rope(q, freqs), atol=1e-5)


def test_autocast_follows_the_stock_policy():
    """Under torch.autocast("blackwell") matrix products and convolutions run in the autocast dtype; losses,
    normalisations and the point-wise functions of the fp32 list run in fp32; softmax / sum / prod / cumsum / norm give
    fp32 results unless the caller names a dtype; mixed inputs promote: the lists torch.autocast("cuda") uses."""
    a, b = torch.randn(4, 8).to(D), torch.randn(8, 8).to(D)
    img, w = torch.randn(2, 8, 6, 6).to(D), torch.randn(8, 8, 3, 3).to(D)
    tgt = torch.zeros(4, dtype=torch.long).to(D)
    for dt in (torch.bfloat16, torch.float16):
        h = a.to(dt)
        with torch.autocast(D, dtype=dt):
            low = [a @ b, F.linear(a, b), F.conv2d(img, w), torch.bmm(a[None], b[None]), torch.addmm(a, a, b), torch.einsum("ij,jk->ik", a, b),
                   F.conv_transpose2d(img, w), nn.LSTMCell(8, 4).to(D)(a)[0], F.scaled_dot_product_attention(a[None], a[None], a[None])]
            f32 = [F.softmax(h, -1), F.log_softmax(h, -1), h.sum(), h.sum(0), h.prod(), h.cumsum(0), h.norm(), torch.linalg.vector_norm(h),
                   F.layer_norm(h, (8,)), F.cross_entropy(h, tgt), F.mse_loss(h, h), h.pow(2.0), h.exp(), h.abs().log(), F.softplus(h),
                   F.group_norm(img.to(dt), 2), F.cosine_similarity(h, h), F.binary_cross_entropy_with_logits(h, h.sigmoid()), F.l1_loss(h, h)]
            promoted = [torch.cat([a, h]), torch.addcmul(a, h, a)]
            kept = [h.sum(dtype=dt), F.softmax(h, -1, dtype=dt), torch.relu(h), h + h]
        assert all(t.dtype == dt for t in low), [t.dtype for t in low]
        assert all(t.dtype == torch.float32 for t in f32), [t.dtype for t in f32]
        assert all(t.dtype == torch.float32 for t in promoted)
        assert all(t.dtype == dt for t in kept)
    assert F.softmax(a.half(), -1).dtype == torch.float16        # outside autocast nothing changes


def test_training_utilities_on_the_device():
    """Activation checkpointing (the dropout mask is replayed from the device generator's saved state), functorch
    transforms, functional_call, weight averaging and parametrizations."""
    from torch.optim.swa_utils import AveragedModel
    from torch.utils.checkpoint import checkpoint

    m = nn.Sequential(nn.Linear(8, 16), nn.Dropout(0.5), nn.ReLU(), nn.Linear(16, 4)).to(D)
    x = torch.randn(5, 8).to(D).requires_grad_()
    for reentrant in (False, True):
        m.zero_grad()
        torch.manual_seed(0)
        a = checkpoint(m, x, use_reentrant=reentrant)
        a.sum().backward()
        g = m[0].weight.grad.clone()
        m.zero_grad()
        torch.manual_seed(0)
        b = m(x)
        b.sum().backward()
        assert torch.allclose(a, b) and torch.allclose(g, m[0].weight.grad)
    xd = x.detach()
    assert torch.allclose(torch.vmap(lambda v: (v * v).sum())(xd).cpu(), (xd ** 2).sum(1).cpu())
    assert torch.allclose(torch.func.grad(lambda v: (v ** 3).sum())(xd).cpu(), (3 * xd ** 2).cpu())
    assert torch.func.functional_call(m.eval(), dict(m.named_parameters()), (x,)).shape == (5, 4)
    avg = AveragedModel(m)
    avg.update_parameters(m)
    avg.update_parameters(m)
    assert all(torch.allclose(p, q) for p, q in zip(avg.module.parameters(), m.parameters()))
    lin = torch.nn.utils.parametrizations.weight_norm(nn.Linear(4, 4).to(D))
    assert lin(torch.randn(2, 4).to(D)).shape == (2, 4)
