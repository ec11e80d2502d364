"""Every model of the zoo runs one forward/backward on a small batch (CPU)."""
import pytest
import torch

from conef_b200 import models

IMAGE_MODELS = [
    ("ResNet20", lambda: models.ResNet20(10), 272474), ("ResNet18", lambda: models.ResNet18(10), 11173962),
    ("ResNet50", lambda: models.ResNet50(10), None), ("WRN-16-2", lambda: models.WideResNet(16, 2, 0.0, 10), None),
    ("VGG11", lambda: models.VGG("VGG11"), None), ("LeNet", lambda: models.LeNet(), None),
    ("densenet_cifar", lambda: models.densenet_cifar(), None), ("MobileNetV2", lambda: models.MobileNetV2(), None),
    ("ShuffleNetV2", lambda: models.ShuffleNetV2(0.5), None), ("ResNeXt29_2x64d", lambda: models.ResNeXt29_2x64d(), None),
]


@pytest.mark.parametrize("name,ctor,params", IMAGE_MODELS, ids=[m[0] for m in IMAGE_MODELS])
def test_image_models_forward_backward(name, ctor, params):
    torch.manual_seed(0)
    net = ctor()
    if params is not None:
        assert sum(p.numel() for p in net.parameters()) == params
    out = net(torch.randn(2, 3, 32, 32))
    assert out.shape == (2, 10)
    out.sum().backward()
    assert all(p.grad is not None for p in net.parameters())


def test_reference_parameter_counts():
    with torch.device("meta"):
        assert sum(p.numel() for p in models.WideResNet28_10(100).parameters()) == 36_546_980
        assert sum(p.numel() for p in models.BertForPreTraining(models.BertConfig.large(30528)).parameters()) == 336_232_258
        assert sum(p.numel() for p in models.RNNModel("LSTM", 33278, 650, 650, 3, 0.5, True).parameters()) == 31_819_578


def test_language_and_translation_models():
    lm = models.RNNModel("GRU", 100, 16, 16, 2, 0.0, tie_weights=True)
    out, h = lm(torch.randint(0, 100, (5, 3)), lm.init_hidden(3))
    assert out.shape == (15, 100)
    tr = models.TransformerModel(100, 16, 2, 32, 2, 0.0)
    assert tr(torch.randint(0, 100, (5, 3))).shape == (5, 3, 100)
    s2s = models.Seq2SeqTransformer(1, 1, 16, 2, 50, 60, 32, 0.0)
    src, tgt = torch.randint(2, 50, (7, 2)), torch.randint(2, 60, (5, 2))
    sm, tm, sp, tp = models.create_mask(src, tgt)
    assert s2s(src, tgt, sm, tm, sp, tp, sp).shape == (5, 2, 60)
    with pytest.raises(ValueError):
        models.RNNModel("LSTM", 10, 8, 16, 1, tie_weights=True)


def test_bert_heads_and_checkpointing():
    cfg = models.BertConfig(200, hidden_size=32, num_hidden_layers=4, num_attention_heads=4, intermediate_size=64)
    net = models.BertForPreTraining(cfg).eval()
    ids = torch.randint(0, 200, (2, 12))
    seg, mask = torch.zeros_like(ids), torch.ones_like(ids)
    a = net(ids, seg, mask)
    net.bert._checkpoint_activations = True
    b = net(ids, seg, mask)
    torch.testing.assert_close(a[0], b[0])
    crit = models.BertPretrainingCriterion(200)
    labels = torch.full((2, 12), -1)
    labels[:, 2] = 7
    loss = crit(a, (labels, torch.tensor([0, 1])))
    assert torch.isfinite(loss)
    assert net.cls.predictions.decoder.weight is net.bert.embeddings.word_embeddings.weight
    assert models.BertForQuestionAnswering(cfg)(ids)[0].shape == (2, 12)
    assert models.BertForSequenceClassification(cfg, 3)(ids).shape == (2, 3)
