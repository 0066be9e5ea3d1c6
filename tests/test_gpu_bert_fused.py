"""Fused transformer pieces on the device: copy-free batched products over head-split views, the fused
dropout + add + LayerNorm block, linears that add their parameter gradients into fp32 buckets with a split-K
weight-gradient GEMM, and the fused BERT layer against the plain module definition."""
import copy
import math

import pytest
import torch
import torch.nn.functional as F

from common import assert_tensors_equal

pytestmark = pytest.mark.gpu
DEV = "blackwell"


@pytest.fixture(scope="module", autouse=True)
def _backend():
    import catch_b200  # noqa: F401

    assert torch.b200.backend_name() == "cuda"
    torch.b200.set_flag("op_trycatch", False)
    yield
    torch.b200.set_flag("op_trycatch", True)


def test_gemm_nd_on_head_split_views():
    from catch_b200.fusion import matmul_nd

    torch.manual_seed(0)
    B, L, h, d = 3, 40, 4, 16
    H = h * d
    qkv = [torch.randn(B, L, H).bfloat16() for _ in range(3)]
    ref = [t.float().view(B, L, h, d).permute(0, 2, 1, 3).detach().requires_grad_() for t in qkv]
    dev_flat = [t.to(DEV).requires_grad_() for t in qkv]
    q, k, v = (t.view(B, L, h, d).permute(0, 2, 1, 3) for t in dev_flat)
    s_ref = ref[0] @ ref[1].transpose(-1, -2) / math.sqrt(d)
    s_dev = matmul_nd(q, k.transpose(-1, -2), 1.0 / math.sqrt(d))
    assert s_dev.shape == (B, h, L, L)
    assert_tensors_equal(s_dev.float(), s_ref, prec=2e-2, use_MSE=True)
    p_ref = torch.softmax(s_ref, -1)
    p_dev = torch.softmax(s_dev.float(), -1).bfloat16()
    c_ref = (p_ref @ ref[2]).permute(0, 2, 1, 3).reshape(B, L, H)
    c_dev = matmul_nd(p_dev, v, 1.0, (L * H, d, H, 1)).permute(0, 2, 1, 3)
    assert c_dev.is_contiguous()                      # written straight into [B, L, h, d] memory
    c_dev = c_dev.reshape(B, L, H)
    assert_tensors_equal(c_dev.float(), c_ref, prec=2e-2, use_MSE=True)
    g = torch.randn(B, L, H)
    c_ref.backward(g); c_dev.backward(g.bfloat16().to(DEV))
    for a, b in zip(ref, dev_flat):
        assert b.grad.shape == (B, L, H) and b.grad.is_contiguous()
        assert_tensors_equal(b.grad.float().view(B, L, h, d).permute(0, 2, 1, 3), a.grad, prec=3e-2, use_MSE=True)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dropout_add_layer_norm(dtype):
    from catch_b200.fusion import dropout_add_layer_norm

    torch.manual_seed(1)
    rows, cols = 300, 768
    norm = torch.nn.LayerNorm(cols)
    norm.weight.data.uniform_(0.5, 1.5); norm.bias.data.normal_()
    nd = copy.deepcopy(norm).to(DEV)
    prec = 3e-3 if dtype == torch.float32 else 2e-2
    # p = 0: exactly residual + h through the layer norm
    h, r = torch.randn(rows, cols), torch.randn(rows, cols)
    hr, rr = h.clone().requires_grad_(), r.clone().requires_grad_()
    hd, rd = h.to(dtype).to(DEV).requires_grad_(), r.to(dtype).to(DEV).requires_grad_()
    yr = norm(rr + hr)
    yd = dropout_add_layer_norm(hd, rd, nd, 0.1, False)
    assert_tensors_equal(yd.float(), yr, prec=prec, use_MSE=True)
    g = torch.randn(rows, cols)
    yr.backward(g); yd.backward(g.to(dtype).to(DEV))
    assert_tensors_equal(hd.grad.float(), hr.grad, prec=prec, use_MSE=True, msg="dh")
    assert_tensors_equal(rd.grad.float(), rr.grad, prec=prec, use_MSE=True, msg="dres")
    assert_tensors_equal(nd.weight.grad, norm.weight.grad, prec=prec, use_MSE=True, msg="dgamma")
    assert_tensors_equal(nd.bias.grad, norm.bias.grad, prec=prec, use_MSE=True, msg="dbeta")
    # p > 0: recover the mask from the op's own output and check forward and backward against it
    p = 0.25
    y, s, mask, mean, rstd = torch.ops.catch_b200.dropout_add_layer_norm(hd.detach(), rd.detach(), nd.weight, nd.bias, p, True, 1e-5)
    bits = mask.cpu().to(torch.int64)
    keep = torch.stack([(bits >> k) & 1 for k in range(4)], -1).reshape(rows, cols).bool()
    assert abs(keep.float().mean().item() - (1 - p)) < 0.01
    s_ref = r.to(dtype).float() + torch.where(keep, h.to(dtype).float() / (1 - p), torch.zeros(()))
    assert_tensors_equal(s.float(), s_ref, prec=prec, use_MSE=True)
    assert_tensors_equal(y.float(), F.layer_norm(s.float().cpu(), (cols,), norm.weight, norm.bias), prec=prec, use_MSE=True)
    ds, dh, dgamma, dbeta = torch.ops.catch_b200.dropout_add_layer_norm_backward(g.to(dtype).to(DEV), s, mask, nd.weight, mean, rstd, p)
    sr = s.detach().float().cpu().clone().requires_grad_(True)
    (ds_ref,) = torch.autograd.grad(F.layer_norm(sr, (cols,), norm.weight.detach(), norm.bias.detach()), sr, g.to(dtype).float())
    assert_tensors_equal(ds.float(), ds_ref, prec=prec, use_MSE=True)
    assert_tensors_equal(dh.float(), torch.where(keep, ds_ref / (1 - p), torch.zeros(())), prec=prec, use_MSE=True)
    # a different call draws a different mask
    _, _, mask2, _, _ = torch.ops.catch_b200.dropout_add_layer_norm(hd.detach(), rd.detach(), nd.weight, nd.bias, p, True, 1e-5)
    assert not torch.equal(mask.cpu(), mask2.cpu())


def test_fused_linear_adds_gradients_into_buckets():
    from catch_b200.fusion import FusedLinear, fuse_linear
    from catch_b200.parallel import FusedDataParallel

    torch.manual_seed(2)
    net = torch.nn.Sequential(torch.nn.Linear(768, 3072), torch.nn.GELU(), torch.nn.Linear(3072, 768))
    ref = copy.deepcopy(net)
    fused = fuse_linear(copy.deepcopy(net)).to(DEV)
    assert all(isinstance(m, FusedLinear) for m in fused if isinstance(m, torch.nn.Linear))
    fdp = FusedDataParallel(fused, "sgd", lr=0.0, bucket_mb=4.0)   # lr 0: the gradients can be inspected through a no_sync pass
    x = torch.randn(4096, 768)
    with fdp.no_sync():
        with torch.autocast(DEV, dtype=torch.bfloat16):
            fdp(x.to(DEV)).float().pow(2).mean().backward()
    ref(x).pow(2).mean().backward()
    for (n, p), (_, q) in zip(ref.named_parameters(), fused.named_parameters()):
        assert q.grad.dtype == torch.float32
        assert_tensors_equal(q.grad, p.grad, prec=3e-2, use_MSE=True, msg=n)   # bf16 operands, fp32 split-K accumulation
    # a second accumulating pass doubles the bucket contents
    before = [q.grad.clone() for q in fused.parameters()]
    with fdp.no_sync():
        with torch.autocast(DEV, dtype=torch.bfloat16):
            fdp(x.to(DEV)).float().pow(2).mean().backward()
    for b, q in zip(before, fused.parameters()):
        assert_tensors_equal(q.grad, 2 * b, prec=1e-3, use_MSE=True)


def test_fused_bert_layer_matches_plain_definition():
    from catch_b200.models.bert import BertConfig, BertForSequenceClassification, FusedBertLayer, fuse_bert

    cfg = BertConfig(vocab_size=200, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, intermediate_size=256,
                     max_position_embeddings=64, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(3)
    plain = BertForSequenceClassification(cfg)
    fused = fuse_bert(copy.deepcopy(plain))
    assert isinstance(fused.layers[0], FusedBertLayer) and set(fused.state_dict()) == set(plain.state_dict())
    plain, fused = plain.to(DEV), fused.to(DEV)
    ids = torch.randint(0, 200, (8, 64)).to(DEV)
    y = torch.randint(0, 2, (8,)).to(DEV)
    losses = []
    for m in (plain, fused):
        with torch.autocast(DEV, dtype=torch.bfloat16):
            loss = F.cross_entropy(m(ids), y)
        loss.backward()
        losses.append(loss.item())
    assert abs(losses[0] - losses[1]) < 2e-2, losses
    bad = {}
    for (n, a), (_, b) in zip(plain.named_parameters(), fused.named_parameters()):
        if n.endswith("attention.key.bias"):
            continue  # softmax is invariant to a shift of all scores of a query: this gradient is rounding noise in both
        ga, gb = a.grad.double().flatten().cpu(), b.grad.double().flatten().cpu()
        cos = (ga @ gb / (ga.norm() * gb.norm() + 1e-30)).item()
        if cos < 0.98:
            bad[n] = round(cos, 4)
    assert not bad, bad
