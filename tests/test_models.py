"""Model definitions on the host-simulated device."""
import torch
import torchvision

import catch_b200  # noqa: F401
from catch_b200.models import BertConfig, BertForSequenceClassification, resnet18, resnet50


def test_resnet_state_dict_matches_torchvision():
    ours, tv = resnet18(), torchvision.models.resnet18()
    assert set(ours.state_dict()) == set(tv.state_dict())
    tv.load_state_dict(ours.state_dict())
    x = torch.randn(2, 3, 64, 64)
    assert torch.allclose(ours.eval()(x), tv.eval()(x), atol=1e-5)
    assert sum(p.numel() for p in resnet50().parameters()) == 25557032


def test_small_bert_trains_on_device():
    cfg = BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                     max_position_embeddings=16, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    ref = BertForSequenceClassification(cfg)
    dev = BertForSequenceClassification(cfg)
    dev.load_state_dict(ref.state_dict())
    dev = dev.to("blackwell")
    ids = torch.randint(0, 100, (3, 16))
    y = torch.tensor([0, 1, 1])
    lr, ld = torch.nn.functional.cross_entropy(ref(ids), y), torch.nn.functional.cross_entropy(dev(ids.to("blackwell")), y.to("blackwell"))
    assert abs(lr.item() - ld.item()) < 1e-4
    lr.backward(); ld.backward()
    for a, b in zip(ref.parameters(), dev.parameters()):
        assert torch.allclose(a.grad, b.grad.cpu(), atol=1e-4)


def test_fused_bert_layers_on_the_host_simulated_device():
    """fuse_bert against the plain layer definitions, with the fused operators on their host paths: products over
    head-split views, dropout + add + LayerNorm in one call, linears whose weight / bias gradients are added into
    the fp32 buckets of FusedDataParallel."""
    import copy

    from catch_b200 import fusion
    from catch_b200.fusion import FusedLinear
    from catch_b200.models.bert import FusedBertLayer, fuse_bert
    from catch_b200.parallel import FusedDataParallel

    cfg = BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                     max_position_embeddings=16, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    ref = BertForSequenceClassification(cfg)
    ids = torch.randint(0, 100, (3, 16))
    att = torch.ones(3, 16); att[1, 10:] = 0
    y = torch.tensor([0, 1, 1])
    with torch.autocast("cpu", dtype=torch.bfloat16):
        loss_ref = torch.nn.functional.cross_entropy(ref(ids, att).float(), y)
    loss_ref.backward()
    fusion.fused_ops_on_host(True)
    try:
        dev = fuse_bert(copy.deepcopy(ref)).to("blackwell")
        dev.zero_grad()
        assert sum(isinstance(m, FusedBertLayer) for m in dev.modules()) == 2
        assert all(isinstance(m, FusedLinear) for m in dev.modules() if isinstance(m, torch.nn.Linear))
        fdp = FusedDataParallel(dev, "adamw", lr=0.0, weight_decay=0.0, bucket_mb=0.01)
        called = []
        orig = torch.ops.catch_b200.linear_backward_fp32w

        def spy(*a):
            called.append((a[6] is not None, a[7] is not None))
            return orig(*a)

        fusion.torch.ops.catch_b200.linear_backward_fp32w = spy
        try:
            with fdp.no_sync():  # gradients stay in the buckets for inspection
                with torch.autocast("blackwell", dtype=torch.bfloat16):
                    loss = torch.nn.functional.cross_entropy(fdp(ids.to("blackwell"), att.to("blackwell")).float(), y.to("blackwell"))
                loss.backward()
        finally:
            fusion.torch.ops.catch_b200.linear_backward_fp32w = orig
        # every linear went through the fused backward and added weight and bias gradients into its bucket
        # (six per layer and the pooler; the two-class classifier is too narrow for the fused path)
        assert len(called) == 2 * 6 + 1 and all(w and b for w, b in called), called
        assert abs(float(loss.detach()) - float(loss_ref)) < 2e-2
        for (n, p), q in zip(ref.named_parameters(), dev.parameters()):
            assert q.grad is not None and q.grad.dtype == torch.float32, n
            if n.endswith("key.bias"):  # the softmax does not depend on it: its gradient is rounding noise around zero
                continue
            err = (q.grad.cpu() - p.grad).norm() / (p.grad.norm() + 1e-8)
            assert err < 6e-2, (n, float(err))      # bf16 activations, different rounding points
        # dropout inside the fused residual block: the kept fraction and the scaling
        h, r = torch.randn(64, 32).to("blackwell"), torch.randn(64, 32).to("blackwell")
        norm = torch.nn.LayerNorm(32).to("blackwell")
        yy, s, mask, mean, rstd = torch.ops.catch_b200.dropout_add_layer_norm(h, r, norm.weight, norm.bias, 0.25, True, 1e-5)
        keep = mask.cpu().bool().reshape(64, 32)
        assert 0.6 < keep.float().mean().item() < 0.9
        assert torch.allclose(s.cpu(), r.cpu() + torch.where(keep, h.cpu() / 0.75, torch.zeros(())), atol=1e-5)
        assert torch.allclose(yy.cpu(), torch.nn.functional.layer_norm(s.cpu(), (32,), norm.weight.cpu(), norm.bias.cpu()), atol=1e-4)
    finally:
        fusion.fused_ops_on_host(False)


def test_lstm_and_gru_run_on_the_device():
    """torch's lstm / gru call fused-cell operators on every non-CPU device, and only CUDA has kernels for them:
    this backend composes them from its element-wise kernels.  Forward, backward and a training step against the CPU."""
    import copy

    torch.manual_seed(0)
    for ctor, shape in ((lambda: torch.nn.LSTM(5, 7, num_layers=2, batch_first=True, bidirectional=True), (3, 6, 5)),
                        (lambda: torch.nn.LSTM(5, 7, bias=False), (6, 3, 5)),
                        (lambda: torch.nn.GRU(5, 7, num_layers=2, bidirectional=True), (6, 3, 5)),
                        (lambda: torch.nn.GRU(5, 7, bias=False, batch_first=True), (3, 6, 5))):
        ref = ctor()
        dev = copy.deepcopy(ref).to("blackwell")
        x = torch.randn(*shape)
        xr, xd = x.clone().requires_grad_(), x.to("blackwell").requires_grad_()
        o_ref, h_ref = ref(xr)
        o_dev, h_dev = dev(xd)
        assert torch.allclose(o_dev.cpu(), o_ref, atol=1e-5)
        h_ref = h_ref if isinstance(h_ref, tuple) else (h_ref,)
        h_dev = h_dev if isinstance(h_dev, tuple) else (h_dev,)
        for a, b in zip(h_dev, h_ref):
            assert torch.allclose(a.cpu(), b, atol=1e-5)
        (o_ref.square().sum() + h_ref[-1].sum()).backward()
        (o_dev.square().sum() + h_dev[-1].sum()).backward()
        assert torch.allclose(xd.grad.cpu(), xr.grad, atol=1e-4)
        for p, q in zip(ref.parameters(), dev.parameters()):
            assert torch.allclose(q.grad.cpu(), p.grad, atol=1e-4)
    # the single-step cells go the same way
    cell, cell_d = torch.nn.LSTMCell(5, 7), None
    cell_d = copy.deepcopy(cell).to("blackwell")
    x = torch.randn(4, 5)
    h, c = cell(x)
    hd, cd = cell_d(x.to("blackwell"))
    assert torch.allclose(hd.cpu(), h, atol=1e-5) and torch.allclose(cd.cpu(), c, atol=1e-5)
