"""BERT encoder with the pre-training heads (masked LM + next-sentence prediction).

Architecture, parameter names and shapes follow the reference's
``examples/BertPretraining/modeling.py`` (``BertConfig`` :189-277, embeddings :335-361,
self-attention :364-417, layer / encoder with activation checkpointing :470-524, heads
:551-599, ``BertModel`` :765-838, ``BertForPreTraining`` :841-902) so that the gradient
buckets — and with them the compression plans — have the reference's shapes: BERT-large
with the vocabulary padded to 30,528 has 336,232,258 parameters.

Differences: attention runs through ``F.scaled_dot_product_attention`` (fused kernels,
additive mask), LayerNorm is ``torch.nn.LayerNorm`` (the reference needs apex for its
fused one), and bf16 comes from autocast instead of apex amp.
"""
import copy
import json
import logging
import math
import os
import re
import shutil
import tarfile
import tempfile

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .layers import LayerNorm, Linear


logger = logging.getLogger(__name__)

CONFIG_NAME = "bert_config.json"
WEIGHTS_NAME = "pytorch_model.bin"
TF_WEIGHTS_NAME = "model.ckpt"


def gelu(x):
    return F.gelu(x)


ACT2FN = {"gelu": gelu, "relu": F.relu, "tanh": torch.tanh, "swish": F.silu, "bias_gelu": gelu}


class BertConfig:
    """Hyper-parameters of a BERT model; constructible from a vocab size or a JSON file."""

    def __init__(self, vocab_size_or_config_json_file=30522, hidden_size=768, num_hidden_layers=12,
                 num_attention_heads=12, intermediate_size=3072, hidden_act="gelu", hidden_dropout_prob=0.1,
                 attention_probs_dropout_prob=0.1, max_position_embeddings=512, type_vocab_size=2,
                 initializer_range=0.02, output_all_encoded_layers=False):
        if isinstance(vocab_size_or_config_json_file, str):
            with open(vocab_size_or_config_json_file, "r", encoding="utf-8") as fh:
                for k, v in json.load(fh).items():
                    setattr(self, k, v)
        elif isinstance(vocab_size_or_config_json_file, int):
            self.vocab_size = vocab_size_or_config_json_file
            self.hidden_size = hidden_size
            self.num_hidden_layers = num_hidden_layers
            self.num_attention_heads = num_attention_heads
            self.hidden_act = hidden_act
            self.intermediate_size = intermediate_size
            self.hidden_dropout_prob = hidden_dropout_prob
            self.attention_probs_dropout_prob = attention_probs_dropout_prob
            self.max_position_embeddings = max_position_embeddings
            self.type_vocab_size = type_vocab_size
            self.initializer_range = initializer_range
            self.output_all_encoded_layers = output_all_encoded_layers
        else:
            raise ValueError("First argument must be a vocabulary size (int) or the path of a JSON config (str)")

    @classmethod
    def from_dict(cls, d):
        cfg = cls(vocab_size_or_config_json_file=-1)
        for k, v in d.items():
            setattr(cfg, k, v)
        return cfg

    @classmethod
    def from_json_file(cls, path):
        with open(path, "r", encoding="utf-8") as fh:
            return cls.from_dict(json.load(fh))

    @classmethod
    def large(cls, vocab_size=30528):
        return cls(vocab_size, hidden_size=1024, num_hidden_layers=24, num_attention_heads=16, intermediate_size=4096)

    @classmethod
    def base(cls, vocab_size=30528):
        return cls(vocab_size)

    def to_dict(self):
        return copy.deepcopy(self.__dict__)

    def to_json_string(self):
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"


class BertEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.word_embeddings = nn.Embedding(config.vocab_size, config.hidden_size)
        self.position_embeddings = nn.Embedding(config.max_position_embeddings, config.hidden_size)
        self.token_type_embeddings = nn.Embedding(config.type_vocab_size, config.hidden_size)
        self.LayerNorm = LayerNorm(config.hidden_size, eps=1e-12)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, input_ids, token_type_ids):
        pos = torch.arange(input_ids.size(1), dtype=torch.long, device=input_ids.device).unsqueeze(0)
        x = self.word_embeddings(input_ids) + self.position_embeddings(pos) + self.token_type_embeddings(token_type_ids)
        return self.dropout(self.LayerNorm(x))


class BertSelfAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        if config.hidden_size % config.num_attention_heads != 0:
            raise ValueError("hidden size must be a multiple of the number of attention heads")
        self.heads = config.num_attention_heads
        self.head_dim = config.hidden_size // config.num_attention_heads
        self.query = Linear(config.hidden_size, config.hidden_size)
        self.key = Linear(config.hidden_size, config.hidden_size)
        self.value = Linear(config.hidden_size, config.hidden_size)
        self.p_drop = config.attention_probs_dropout_prob

    def forward(self, x, mask):
        b, s, _ = x.shape
        split = lambda t: t.view(b, s, self.heads, self.head_dim).transpose(1, 2)
        ctx = F.scaled_dot_product_attention(split(self.query(x)), split(self.key(x)), split(self.value(x)),
                                             attn_mask=mask, dropout_p=self.p_drop if self.training else 0.0)
        return ctx.transpose(1, 2).reshape(b, s, self.heads * self.head_dim)


class BertSelfOutput(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = Linear(config.hidden_size, config.hidden_size)
        self.LayerNorm = LayerNorm(config.hidden_size, eps=1e-12)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, h, residual):
        return self.LayerNorm(self.dropout(self.dense(h)) + residual)


class BertAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.self = BertSelfAttention(config)
        self.output = BertSelfOutput(config)

    def forward(self, x, mask):
        return self.output(self.self(x, mask), x)


class BertIntermediate(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = Linear(config.hidden_size, config.intermediate_size)
        self.act = ACT2FN[config.hidden_act]

    def forward(self, x):
        return self.act(self.dense(x))


class BertOutput(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = Linear(config.intermediate_size, config.hidden_size)
        self.LayerNorm = LayerNorm(config.hidden_size, eps=1e-12)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, h, residual):
        return self.LayerNorm(self.dropout(self.dense(h)) + residual)


class BertLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.attention = BertAttention(config)
        self.intermediate = BertIntermediate(config)
        self.output = BertOutput(config)

    def forward(self, x, mask):
        a = self.attention(x, mask)
        return self.output(self.intermediate(a), a)


class BertEncoder(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layer = nn.ModuleList([BertLayer(config) for _ in range(config.num_hidden_layers)])
        self.output_all_encoded_layers = config.output_all_encoded_layers

    def _checkpointed(self, x, mask):
        # sqrt(L) chunks of layers: only chunk boundaries keep their activations
        n = len(self.layer)
        chunk = max(1, int(math.ceil(math.sqrt(n))))
        for lo in range(0, n, chunk):
            def run(h, lo=lo):
                for layer in self.layer[lo : lo + chunk]:
                    h = layer(h, mask)
                return h
            x = checkpoint(run, x, use_reentrant=False)
        return x

    def forward(self, x, mask, checkpoint_activations=False):
        if checkpoint_activations:
            return [self._checkpointed(x, mask)]
        outs = []
        for layer in self.layer:
            x = layer(x, mask)
            if self.output_all_encoded_layers:
                outs.append(x)
        if not self.output_all_encoded_layers:
            outs.append(x)
        return outs


class BertPooler(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.hidden_size)

    def forward(self, h):
        return torch.tanh(self.dense(h[:, 0]))


class BertPredictionHeadTransform(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.hidden_size)
        self.act = ACT2FN[config.hidden_act]
        self.LayerNorm = LayerNorm(config.hidden_size, eps=1e-12)

    def forward(self, h):
        return self.LayerNorm(self.act(self.dense(h)))


class BertLMPredictionHead(nn.Module):
    """Decoder tied to the word embeddings plus an output-only bias."""

    def __init__(self, config, embedding_weights):
        super().__init__()
        self.transform = BertPredictionHeadTransform(config)
        self.decoder = nn.Linear(embedding_weights.size(1), embedding_weights.size(0), bias=False)
        self.decoder.weight = embedding_weights
        self.bias = nn.Parameter(torch.zeros(embedding_weights.size(0)))

    def forward(self, h):
        return self.decoder(self.transform(h)) + self.bias


class BertPreTrainingHeads(nn.Module):
    def __init__(self, config, embedding_weights):
        super().__init__()
        self.predictions = BertLMPredictionHead(config, embedding_weights)
        self.seq_relationship = nn.Linear(config.hidden_size, 2)

    def forward(self, sequence_output, pooled_output):
        return self.predictions(sequence_output), self.seq_relationship(pooled_output)


class BertPreTrainedModel(nn.Module):
    def __init__(self, config):
        super().__init__()
        if not isinstance(config, BertConfig):
            raise ValueError("config must be a BertConfig")
        self.config = config

    def init_bert_weights(self, module):
        if isinstance(module, (nn.Linear, nn.Embedding)):
            module.weight.data.normal_(mean=0.0, std=self.config.initializer_range)
        elif isinstance(module, nn.LayerNorm):
            module.bias.data.zero_()
            module.weight.data.fill_(1.0)
        if isinstance(module, nn.Linear) and module.bias is not None:
            module.bias.data.zero_()

    def checkpoint_activations(self, val):
        def _apply(m):
            if hasattr(m, "_checkpoint_activations"):
                m._checkpoint_activations = val
        self.apply(_apply)

    def save_pretrained(self, directory: str) -> None:
        """Write ``bert_config.json`` and ``pytorch_model.bin``, the layout :meth:`from_pretrained` reads."""
        os.makedirs(directory, exist_ok=True)
        with open(os.path.join(directory, CONFIG_NAME), "w", encoding="utf-8") as f:
            f.write(self.config.to_json_string())
        torch.save(self.state_dict(), os.path.join(directory, WEIGHTS_NAME))

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, state_dict=None, cache_dir=None, from_tf=False,
                        *inputs, **kwargs):
        """Build ``cls`` from a saved model (reference: ``modeling.py:641-762``).

        ``pretrained_model_name_or_path``: a directory holding ``bert_config.json`` and
        ``pytorch_model.bin`` (or, with ``from_tf``, TensorFlow-named weights: ``model.ckpt`` read with
        TensorFlow when it is installed, or ``model.ckpt.npz`` holding the same variables as arrays), a
        ``.tar.gz`` archive of such a directory, or a URL / name that the local file cache
        (:mod:`conef_b200.utils.file_cache`) resolves.  Old checkpoints' ``gamma`` / ``beta`` LayerNorm
        names are renamed; a state dict saved from a model with a ``bert.`` prefix loads into a bare
        ``BertModel``; weights the checkpoint lacks (a new task head) keep their initialisation and
        are logged, mismatched shapes raise.  Extra arguments go to the constructor (``num_labels`` ...).
        """
        from ..utils.file_cache import cached_path

        resolved = cached_path(pretrained_model_name_or_path, cache_dir=cache_dir)
        tempdir = None
        if os.path.isdir(resolved):
            folder = resolved
        else:
            tempdir = tempfile.mkdtemp()
            with tarfile.open(resolved, "r:*") as archive:
                archive.extractall(tempdir, filter="data")
            folder = tempdir
            entries = os.listdir(folder)
            if CONFIG_NAME not in entries and len(entries) == 1 and os.path.isdir(os.path.join(folder, entries[0])):
                folder = os.path.join(folder, entries[0])
        try:
            config = BertConfig.from_json_file(os.path.join(folder, CONFIG_NAME))
            model = cls(config, *inputs, **kwargs)
            if from_tf:
                return load_tf_weights_in_bert(model, os.path.join(folder, TF_WEIGHTS_NAME))
            if state_dict is None:
                state_dict = torch.load(os.path.join(folder, WEIGHTS_NAME), map_location="cpu", weights_only=True)
        finally:
            if tempdir:
                shutil.rmtree(tempdir, ignore_errors=True)
        renamed = {}
        for key, value in state_dict.items():
            new = re.sub(r"(^|\.)gamma$", r"\1weight", key)
            new = re.sub(r"(^|\.)beta$", r"\1bias", new)
            renamed[new] = value
        if not hasattr(model, "bert") and any(k.startswith("bert.") for k in renamed):
            renamed = {k[len("bert."):]: v for k, v in renamed.items() if k.startswith("bert.")}
        result = model.load_state_dict(renamed, strict=False)
        if result.missing_keys:
            logger.info("Weights of %s not initialized from pretrained model: %s", cls.__name__, result.missing_keys)
        if result.unexpected_keys:
            logger.info("Weights from pretrained model not used in %s: %s", cls.__name__, result.unexpected_keys)
        return model


def load_tf_weights_in_bert(model, tf_checkpoint_path):
    """Copy TensorFlow-named BERT variables into ``model`` (reference: ``modeling.py:59-117``).

    ``tf_checkpoint_path``: a mapping ``{variable name: array}``, an ``.npz`` file of such arrays (also
    tried as ``<path>.npz``), or a TensorFlow checkpoint prefix, which needs TensorFlow.  Naming
    rules: path components separated by ``/``; ``layer_7`` indexes a module list; ``kernel`` is a
    Linear weight stored transposed; ``gamma`` / ``beta`` are LayerNorm weight / bias; ``output_bias`` /
    ``output_weights`` are a head's bias / weight; a trailing ``*_embeddings`` names an Embedding's
    weight; optimizer slots (``adam_m``, ``adam_v``) and ``global_step`` are skipped."""
    import numpy as np

    if isinstance(tf_checkpoint_path, dict):
        variables = dict(tf_checkpoint_path)
    else:
        path = os.fspath(tf_checkpoint_path)
        npz = path if path.endswith(".npz") else path + ".npz"
        if os.path.exists(npz):
            with np.load(npz) as z:
                variables = {k: z[k] for k in z.files}
        else:
            try:
                import tensorflow as tf
            except ImportError as exc:
                raise ImportError("reading a TensorFlow checkpoint needs TensorFlow; export the variables to "
                                  f"{npz} (name -> array) to load them without it") from exc
            variables = {name: tf.train.load_variable(path, name) for name, _ in tf.train.list_variables(path)}
    for name, array in variables.items():
        parts = name.split("/")
        if any(p in ("adam_v", "adam_m", "global_step") for p in parts):
            continue
        pointer = model
        for part in parts:
            m = re.fullmatch(r"([A-Za-z]+)_(\d+)", part)
            key, index = (m.group(1), int(m.group(2))) if m else (part, None)
            if key in ("kernel", "gamma", "output_weights"):
                pointer = getattr(pointer, "weight")
            elif key in ("output_bias", "beta"):
                pointer = getattr(pointer, "bias")
            else:
                pointer = getattr(pointer, key)
            if index is not None:
                pointer = pointer[index]
        if parts[-1].endswith("_embeddings"):
            pointer = getattr(pointer, "weight")
        elif parts[-1] == "kernel":
            array = np.ascontiguousarray(np.transpose(array))
        if tuple(pointer.shape) != tuple(array.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(array.shape)} does not match {tuple(pointer.shape)}")
        with torch.no_grad():
            pointer.copy_(torch.from_numpy(np.asarray(array)).to(pointer.dtype))
    return model


def tf_variable_names(model):
    """``{TensorFlow variable name: array}`` of ``model``'s parameters: the inverse of the naming rules
    of :func:`load_tf_weights_in_bert` (to export weights, and to test the loader)."""
    out = {}
    modules = dict(model.named_modules())
    for pname, p in model.named_parameters():
        mod_name, _, leaf = pname.rpartition(".")
        mod = modules[mod_name]
        parts = mod_name.split(".") if mod_name else []
        tf_parts, i = [], 0
        while i < len(parts):               # "layer", "7" -> "layer_7"
            if i + 1 < len(parts) and parts[i + 1].isdigit():
                tf_parts.append(f"{parts[i]}_{parts[i + 1]}")
                i += 2
            else:
                tf_parts.append(parts[i])
                i += 1
        arr = p.detach().cpu().numpy()
        if isinstance(mod, nn.Embedding):
            out["/".join(tf_parts)] = arr
        elif isinstance(mod, nn.LayerNorm):
            out["/".join(tf_parts + ["gamma" if leaf == "weight" else "beta"])] = arr
        elif isinstance(mod, nn.Linear) and leaf == "weight":
            out["/".join(tf_parts + ["kernel"])] = arr.T.copy()
        else:
            out["/".join(tf_parts + [leaf])] = arr
    return out


class BertModel(BertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.embeddings = BertEmbeddings(config)
        self.encoder = BertEncoder(config)
        self.pooler = BertPooler(config)
        self._checkpoint_activations = False
        self.apply(self.init_bert_weights)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None):
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        if token_type_ids is None:
            token_type_ids = torch.zeros_like(input_ids)
        emb = self.embeddings(input_ids, token_type_ids)
        # additive mask broadcast over heads and query positions: 0 keep, -10000 drop
        ext = (1.0 - attention_mask[:, None, None, :].to(emb.dtype)) * -10000.0
        layers = self.encoder(emb, ext, checkpoint_activations=self._checkpoint_activations)
        pooled = self.pooler(layers[-1])
        return (layers if self.config.output_all_encoded_layers else layers[-1]), pooled


class BertForPreTraining(BertPreTrainedModel):
    """Returns ``(prediction_scores [B, S, V], seq_relationship_score [B, 2])``."""

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config)
        self.cls = BertPreTrainingHeads(config, self.bert.embeddings.word_embeddings.weight)
        self.apply(self.init_bert_weights)

    def forward(self, input_ids, token_type_ids, attention_mask):
        seq, pooled = self.bert(input_ids, token_type_ids, attention_mask)
        if isinstance(seq, list):
            seq = seq[-1]
        return self.cls(seq, pooled)


def _last(seq):
    return seq[-1] if isinstance(seq, list) else seq


class BertForMaskedLM(BertPreTrainedModel):
    """Masked-LM logits ``[B, S, V]``, or the loss when ``masked_lm_labels`` (-1 = ignored) is given
    (reference: ``modeling.py:905-965``)."""

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config)
        self.cls = BertLMPredictionHead(config, self.bert.embeddings.word_embeddings.weight)
        self.apply(self.init_bert_weights)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None, masked_lm_labels=None):
        seq, _ = self.bert(input_ids, token_type_ids, attention_mask)
        scores = self.cls(_last(seq))
        if masked_lm_labels is None:
            return scores
        return F.cross_entropy(scores.view(-1, self.config.vocab_size).float(), masked_lm_labels.view(-1),
                               ignore_index=-1)


class BertForNextSentencePrediction(BertPreTrainedModel):
    """Is-next / not-next logits ``[B, 2]`` from the pooled output, or the loss when
    ``next_sentence_label`` is given (reference: ``modeling.py:968-1027``)."""

    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config)
        self.cls = BertOnlyNSPHead(config)
        self.apply(self.init_bert_weights)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None, next_sentence_label=None):
        _, pooled = self.bert(input_ids, token_type_ids, attention_mask)
        score = self.cls(pooled)
        if next_sentence_label is None:
            return score
        return F.cross_entropy(score.view(-1, 2).float(), next_sentence_label.view(-1), ignore_index=-1)


class BertOnlyNSPHead(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.seq_relationship = nn.Linear(config.hidden_size, 2)

    def forward(self, pooled_output):
        return self.seq_relationship(pooled_output)


class BertForMultipleChoice(BertPreTrainedModel):
    """Inputs ``[B, num_choices, S]``; one score per choice from a shared encoder and a
    ``hidden -> 1`` classifier; logits ``[B, num_choices]`` or the loss (reference: ``modeling.py:1093-1160``)."""

    def __init__(self, config, num_choices=2):
        super().__init__(config)
        self.num_choices = num_choices
        self.bert = BertModel(config)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)
        self.classifier = nn.Linear(config.hidden_size, 1)
        self.apply(self.init_bert_weights)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None, labels=None):
        flat = lambda t: None if t is None else t.reshape(-1, t.size(-1))
        _, pooled = self.bert(flat(input_ids), flat(token_type_ids), flat(attention_mask))
        logits = self.classifier(self.dropout(pooled)).view(-1, self.num_choices)
        if labels is None:
            return logits
        return F.cross_entropy(logits.float(), labels)


class BertForTokenClassification(BertPreTrainedModel):
    """A label per token: logits ``[B, S, num_labels]``, or the loss over the positions the attention
    mask keeps (reference: ``modeling.py:1163-1228``)."""

    def __init__(self, config, num_labels=2):
        super().__init__(config)
        self.num_labels = num_labels
        self.bert = BertModel(config)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)
        self.classifier = nn.Linear(config.hidden_size, num_labels)
        self.apply(self.init_bert_weights)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None, labels=None):
        seq, _ = self.bert(input_ids, token_type_ids, attention_mask)
        logits = self.classifier(self.dropout(_last(seq)))
        if labels is None:
            return logits
        flat_logits, flat_labels = logits.view(-1, self.num_labels).float(), labels.view(-1)
        if attention_mask is not None:
            active = attention_mask.view(-1) == 1
            flat_logits, flat_labels = flat_logits[active], flat_labels[active]
        return F.cross_entropy(flat_logits, flat_labels)


class BertForSequenceClassification(BertPreTrainedModel):
    def __init__(self, config, num_labels=2):
        super().__init__(config)
        self.bert = BertModel(config)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)
        self.classifier = nn.Linear(config.hidden_size, num_labels)
        self.apply(self.init_bert_weights)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None):
        _, pooled = self.bert(input_ids, token_type_ids, attention_mask)
        return self.classifier(self.dropout(pooled))


class BertForQuestionAnswering(BertPreTrainedModel):
    def __init__(self, config):
        super().__init__(config)
        self.bert = BertModel(config)
        self.qa_outputs = nn.Linear(config.hidden_size, 2)
        self.apply(self.init_bert_weights)

    def forward(self, input_ids, token_type_ids=None, attention_mask=None):
        seq, _ = self.bert(input_ids, token_type_ids, attention_mask)
        logits = self.qa_outputs(seq[-1] if isinstance(seq, list) else seq)
        start, end = logits.split(1, dim=-1)
        return start.squeeze(-1), end.squeeze(-1)


class BertPretrainingCriterion(nn.Module):
    """Masked-LM cross entropy (labels -1 are ignored) plus next-sentence cross entropy
    (reference: run_pretraining_conef.py:134-144)."""

    def __init__(self, vocab_size):
        super().__init__()
        self.vocab_size = vocab_size

    def forward(self, outputs, targets):
        prediction_scores, seq_relationship_score = outputs
        masked_lm_labels, next_sentence_labels = targets
        mlm = F.cross_entropy(prediction_scores.view(-1, self.vocab_size).float(), masked_lm_labels.view(-1),
                              ignore_index=-1)
        nsp = F.cross_entropy(seq_relationship_score.view(-1, 2).float(), next_sentence_labels.view(-1))
        return mlm + nsp
