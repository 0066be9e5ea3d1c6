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
