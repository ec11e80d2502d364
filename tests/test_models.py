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


def _tiny_bert_config():
    from conef_b200 import models
    return models.BertConfig(96, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64,
                             max_position_embeddings=40)


def test_bert_task_heads_shapes_and_losses():
    """Next-sentence, multiple-choice and token-classification heads (reference modeling.py:968-1228)."""
    import torch
    from conef_b200 import models

    cfg = _tiny_bert_config()
    ids = torch.randint(0, 96, (3, 10))
    seg = torch.randint(0, 2, (3, 10))
    mask = torch.ones(3, 10, dtype=torch.long)
    mask[1, 7:] = 0
    nsp = models.BertForNextSentencePrediction(cfg).eval()
    assert nsp(ids, seg, mask).shape == (3, 2)
    assert nsp(ids, seg, mask, next_sentence_label=torch.tensor([0, 1, 1])).dim() == 0
    mc = models.BertForMultipleChoice(cfg, num_choices=4).eval()
    ids4 = torch.randint(0, 96, (3, 4, 10))
    out = mc(ids4, torch.zeros_like(ids4), torch.ones_like(ids4))
    assert out.shape == (3, 4)
    mc(ids4, torch.zeros_like(ids4), torch.ones_like(ids4), labels=torch.tensor([0, 3, 2])).backward()
    tok = models.BertForTokenClassification(cfg, num_labels=5).eval()
    assert tok(ids, seg, mask).shape == (3, 10, 5)
    labels = torch.randint(0, 5, (3, 10))
    full = tok(ids, seg, mask, labels=labels)
    labels2 = labels.clone()
    labels2[1, 7:] = (labels2[1, 7:] + 1) % 5           # labels under the padding do not count
    torch.testing.assert_close(full, tok(ids, seg, mask, labels=labels2))
    mlm = models.BertForMaskedLM(cfg).eval()
    lab = torch.full((3, 10), -1)
    lab[0, 2] = 5
    assert mlm(ids, seg, mask, masked_lm_labels=lab).dim() == 0


def test_bert_from_pretrained_directory_archive_and_prefixes(tmp_path):
    """save_pretrained -> from_pretrained from a directory and a .tar.gz, LayerNorm gamma/beta names,
    a pre-training checkpoint loaded into a bare encoder and into a model with a new head."""
    import tarfile
    import torch
    from conef_b200 import models

    torch.manual_seed(0)
    src = models.BertForPreTraining(_tiny_bert_config())
    src.save_pretrained(str(tmp_path / "m"))
    again = models.BertForPreTraining.from_pretrained(str(tmp_path / "m"))
    for (k, a), (_, b) in zip(src.state_dict().items(), again.state_dict().items()):
        assert torch.equal(a, b), k
    with tarfile.open(tmp_path / "m.tar.gz", "w:gz") as tar:
        for name in ("bert_config.json", "pytorch_model.bin"):
            tar.add(tmp_path / "m" / name, arcname=name)
    from_tar = models.BertModel.from_pretrained(str(tmp_path / "m.tar.gz"))       # "bert." prefix stripped
    assert torch.equal(from_tar.embeddings.word_embeddings.weight, src.bert.embeddings.word_embeddings.weight)
    old_style = {k.replace("LayerNorm.weight", "LayerNorm.gamma").replace("LayerNorm.bias", "LayerNorm.beta"): v
                 for k, v in src.state_dict().items()}
    head = models.BertForSequenceClassification.from_pretrained(str(tmp_path / "m"), state_dict=old_style, num_labels=3)
    assert head.classifier.weight.shape == (3, 32)
    assert torch.equal(head.bert.encoder.layer[1].output.LayerNorm.weight, src.bert.encoder.layer[1].output.LayerNorm.weight)
    import pytest
    with pytest.raises(EnvironmentError):
        models.BertModel.from_pretrained(str(tmp_path / "missing"))


def test_bert_tensorflow_named_weights_round_trip(tmp_path):
    """The TensorFlow naming rules (kernel = transposed weight, gamma/beta, layer_N, *_embeddings) both ways."""
    import numpy as np
    import torch
    from conef_b200 import models

    torch.manual_seed(1)
    src = models.BertForPreTraining(_tiny_bert_config())
    variables = models.tf_variable_names(src)
    assert "bert/encoder/layer_1/attention/self/query/kernel" in variables
    assert "bert/embeddings/word_embeddings" in variables and "bert/embeddings/LayerNorm/gamma" in variables
    variables["bert/encoder/layer_0/output/dense/kernel/adam_m"] = np.zeros((64, 32), np.float32)   # optimizer slot: skipped
    variables["global_step"] = np.zeros((), np.int64)
    dst = models.BertForPreTraining(_tiny_bert_config())
    models.load_tf_weights_in_bert(dst, variables)
    for (k, a), (_, b) in zip(src.state_dict().items(), dst.state_dict().items()):
        assert torch.equal(a, b), k
    (tmp_path / "tf").mkdir()
    np.savez(tmp_path / "tf" / "model.ckpt.npz", **{k: v for k, v in variables.items() if "adam" not in k})
    (tmp_path / "tf" / "bert_config.json").write_text(src.config.to_json_string())
    via = models.BertForPreTraining.from_pretrained(str(tmp_path / "tf"), from_tf=True)
    assert torch.equal(via.cls.predictions.transform.dense.weight, src.cls.predictions.transform.dense.weight)
    bad = dict(variables)
    bad["bert/pooler/dense/kernel"] = np.zeros((3, 3), np.float32)
    import pytest
    with pytest.raises(ValueError):
        models.load_tf_weights_in_bert(models.BertForPreTraining(_tiny_bert_config()), bad)


def test_file_cache_is_local_first(tmp_path):
    from conef_b200.utils import file_cache as fc

    f = tmp_path / "vocab.txt"
    f.write_text("[PAD]\n[UNK]\n")
    assert fc.cached_path(str(f)) == str(f)
    url = "https://example.invalid/models/bert-tiny/vocab.txt"
    cache = str(tmp_path / "cache")
    with __import__("pytest").raises(EnvironmentError):
        fc.cached_path(url, cache_dir=cache)                   # not cached, and no network
    stored = fc.add_to_cache(url, str(f), etag='"abc"', cache_dir=cache)
    assert fc.cached_path(url, cache_dir=cache) == stored
    import os
    assert fc.filename_to_url(os.path.basename(stored), cache) == (url, '"abc"')
    assert fc.url_to_filename(url, '"abc"') == os.path.basename(stored)
    with __import__("pytest").raises(EnvironmentError):
        fc.cached_path(str(tmp_path / "nope.txt"))
