"""Export a BERT question-answering model into a Triton Inference Server model repository.

Counterpart of the reference's ``examples/BertPretraining/triton/deployer.py`` and
``triton/deployer_lib.py`` (TorchScript or ONNX export ``deployer_lib.py:330-470``, generated
``config.pbtxt`` ``:285-328``, exported-against-eager check with L-infinity errors ``:264-283``).
The layout written is the one the server reads::

    <repository>/<model_name>/config.pbtxt
    <repository>/<model_name>/<version>/model.pt      (TorchScript)  or  model.onnx

Nothing here needs a server: ``client.py`` beside this file can load the same repository
in-process, so the export is checked end to end on any machine.

    python examples/bert_pretraining/deploy/export.py --bert_model base --init_checkpoint ckpt.pt \
        --repository /models --model_name bert_qa --format ts-trace --max_seq_length 384 --batch_size 8
"""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", ".."))

from conef_b200 import models  # noqa: E402

TRITON_TYPES = {torch.int64: "TYPE_INT64", torch.int32: "TYPE_INT32", torch.float32: "TYPE_FP32",
                torch.float16: "TYPE_FP16", torch.bfloat16: "TYPE_BF16", torch.bool: "TYPE_BOOL"}
FORMATS = {"ts-trace": ("pytorch_libtorch", "model.pt"), "onnx": ("onnxruntime_onnx", "model.onnx")}


def as_tuple(out):
    return (out,) if torch.is_tensor(out) else tuple(out)


def dynamic_dims(tensor_lists):
    """Per tensor position, the dimensions after the batch axis, with -1 where the sample batches
    disagree (``[(ids[2,16], ...), (ids[4,24], ...)]`` gives ``[[-1], ...]``)."""
    dims = [list(t.shape[1:]) for t in tensor_lists[0]]
    for tensors in tensor_lists[1:]:
        if len(tensors) != len(dims):
            raise ValueError("sample batches differ in their number of tensors")
        for d, t in zip(dims, tensors):
            if t.dim() - 1 != len(d):
                raise ValueError("sample batches differ in rank")
            for j, size in enumerate(t.shape[1:]):
                if d[j] != size:
                    d[j] = -1
    return dims


def _io_block(kind, prefix, dims, dtypes):
    items = []
    for i, (d, dt) in enumerate(zip(dims, dtypes)):
        items.append("  {\n    name: \"%s__%d\"\n    data_type: %s\n    dims: [%s]\n  }"
                     % (prefix, i, TRITON_TYPES[dt], ", ".join(str(x) for x in d)))
    return "%s [\n%s\n]" % (kind, ",\n".join(items))


def config_pbtxt(name, platform, max_batch_size, in_dims, in_types, out_dims, out_types, instances=1,
                 on_gpu=True, dynamic_batching_delay_us=0, preferred_batch_sizes=()):
    """Text of ``config.pbtxt``.  Tensor names follow the libtorch backend's positional convention
    (``input__0`` ..., ``output__0`` ...); the batch axis is implied by ``max_batch_size``."""
    parts = ["name: \"%s\"" % name, "platform: \"%s\"" % platform, "max_batch_size: %d" % max_batch_size,
             _io_block("input", "input", in_dims, in_types), _io_block("output", "output", out_dims, out_types),
             "instance_group [\n  {\n    count: %d\n    kind: %s\n  }\n]" % (instances, "KIND_GPU" if on_gpu else "KIND_CPU")]
    if dynamic_batching_delay_us > 0 or preferred_batch_sizes:
        body = []
        if preferred_batch_sizes:
            body.append("  preferred_batch_size: [%s]" % ", ".join(str(b) for b in preferred_batch_sizes))
        body.append("  max_queue_delay_microseconds: %d" % dynamic_batching_delay_us)
        parts.append("dynamic_batching {\n%s\n}" % "\n".join(body))
    return "\n".join(parts) + "\n"


def to_torchscript(model, sample):
    """Trace one forward pass.  The trace is shape-generic for this model (no Python control flow depends
    on the sizes; checked below on batches of other shapes).  ``torch.jit.script``, which the reference
    also offers (``deployer_lib.py:352-376``), is not: the model is written outside the scriptable subset
    of Python, and under ``no_grad`` its custom layers are the stock ones, so tracing loses nothing."""
    model.eval()
    with torch.no_grad():
        return torch.jit.trace(model, tuple(sample), check_trace=False)


def linf_report(reference_outputs, exported_outputs):
    """Largest absolute difference per output tensor over all sample batches, with its statistics."""
    errs = []
    for a, b in zip(reference_outputs, exported_outputs):
        for x, y in zip(a, b):
            errs.append(float((x.float() - y.float()).abs().max()))
    rep = {"tensors_compared": len(errs), "max_linf": max(errs), "mean_linf": statistics.mean(errs)}
    rep["stdev_linf"] = statistics.stdev(errs) if len(errs) > 1 else 0.0
    return rep


def export_repository(model, sample_batches, repository, name, fmt="ts-trace", version=1, max_batch_size=8,
                      instances=1, dynamic_batching_delay_us=0, preferred_batch_sizes=(), tolerance=None):
    """Write ``<repository>/<name>`` and return the report (paths, shapes, L-infinity check).

    ``sample_batches``: a list of input tuples on the model's device; the first is the tracing example,
    all of them are replayed through the exported model and compared with the eager one.  At least two
    batches of different sequence lengths make the sequence axis dynamic in ``config.pbtxt``."""
    if fmt not in FORMATS:
        raise ValueError(f"unknown format {fmt!r}; one of {sorted(FORMATS)}")
    platform, filename = FORMATS[fmt]
    model.eval()
    device = sample_batches[0][0].device
    with torch.no_grad():
        eager_out = [as_tuple(model(*b)) for b in sample_batches]
    model_dir = os.path.join(repository, name)
    version_dir = os.path.join(model_dir, str(version))
    os.makedirs(version_dir, exist_ok=True)
    target = os.path.join(version_dir, filename)
    if fmt == "onnx":
        n_in, n_out = len(sample_batches[0]), len(eager_out[0])
        in_names = [f"input__{i}" for i in range(n_in)]
        out_names = [f"output__{i}" for i in range(n_out)]
        axes = {n: {0: "batch", **{j + 1: f"{n}_d{j}" for j in range(sample_batches[0][i].dim() - 1)}}
                for i, n in enumerate(in_names)}
        axes.update({n: {0: "batch", **{j + 1: f"{n}_d{j}" for j in range(eager_out[0][i].dim() - 1)}}
                     for i, n in enumerate(out_names)})
        try:
            torch.onnx.export(model, tuple(sample_batches[0]), target, input_names=in_names, output_names=out_names,
                              dynamic_axes=axes, opset_version=17, dynamo=False)
        except Exception as e:      # the exporter needs the onnx package of the image
            raise RuntimeError(f"ONNX export is not available in this environment: {e}") from e
        exported_out = None         # checked by the serving runtime, not here: no ONNX runtime is assumed
    else:
        ts = to_torchscript(model, sample_batches[0])
        ts.save(target)
        loaded = torch.jit.load(target, map_location=device)
        with torch.no_grad():
            exported_out = [as_tuple(loaded(*b)) for b in sample_batches]
    in_dims = dynamic_dims([tuple(b) for b in sample_batches])
    out_dims = dynamic_dims(eager_out)
    cfg = config_pbtxt(name, platform, max_batch_size, in_dims, [t.dtype for t in sample_batches[0]], out_dims,
                       [t.dtype for t in eager_out[0]], instances, device.type == "cuda",
                       dynamic_batching_delay_us, preferred_batch_sizes)
    with open(os.path.join(model_dir, "config.pbtxt"), "w") as f:
        f.write(cfg)
    report = {"model": target, "config": os.path.join(model_dir, "config.pbtxt"), "format": fmt,
              "input_dims": in_dims, "output_dims": out_dims, "max_batch_size": max_batch_size}
    if exported_out is not None:
        report["check"] = linf_report(eager_out, exported_out)
        if tolerance is not None and report["check"]["max_linf"] > tolerance:
            raise RuntimeError(f"exported model differs from the eager one: {report['check']}")
    return report


def build_model(args, device):
    if args.config_file:
        cfg = models.BertConfig.from_json_file(args.config_file)
    elif args.bert_model == "large":
        cfg = models.BertConfig.large()
    elif args.bert_model == "base":
        cfg = models.BertConfig.base()
    else:
        cfg = models.BertConfig(args.tiny_vocab, hidden_size=128, num_hidden_layers=2, num_attention_heads=4,
                                intermediate_size=512)
    net = models.BertForQuestionAnswering(cfg)
    if args.init_checkpoint:
        sd = torch.load(args.init_checkpoint, map_location="cpu")
        missing, unexpected = net.load_state_dict(sd.get("model", sd), strict=False)
        print(f"loaded {args.init_checkpoint}: {len(missing)} missing, {len(unexpected)} unexpected keys",
              file=sys.stderr)
    net = net.to(device).eval()
    if args.fp16:
        net = net.half()
    return net, cfg


def sample_inputs(cfg, batch, seq, device, seed):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, cfg.vocab_size, (batch, seq), generator=g)
    seg = (torch.arange(seq)[None, :] >= seq // 3).long().expand(batch, seq).contiguous()
    mask = torch.ones(batch, seq, dtype=torch.long)
    mask[:, seq - seq // 8:] = 0
    return tuple(t.to(device) for t in (ids, seg, mask))


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--repository", required=True, help="model repository directory of the server")
    p.add_argument("--model_name", default="bert_qa")
    p.add_argument("--version", type=int, default=1)
    p.add_argument("--format", default="ts-trace", choices=sorted(FORMATS))
    p.add_argument("--bert_model", default="base", choices=["large", "base", "tiny"])
    p.add_argument("--tiny_vocab", type=int, default=1000)
    p.add_argument("--config_file", default=None)
    p.add_argument("--init_checkpoint", default=None, help="checkpoint with a 'model' state dict; random weights without")
    p.add_argument("--max_seq_length", type=int, default=384)
    p.add_argument("--batch_size", type=int, default=8, help="max_batch_size of the served model")
    p.add_argument("--fp16", action="store_true")
    p.add_argument("--instances", type=int, default=1)
    p.add_argument("--dynamic_batching_delay_us", type=int, default=0)
    p.add_argument("--preferred_batch_sizes", type=int, nargs="*", default=[])
    p.add_argument("--tolerance", type=float, default=None, help="fail when the L-infinity error is larger")
    p.add_argument("--no_cuda", action="store_true")
    p.add_argument("--seed", type=int, default=1)
    args = p.parse_args(argv)
    torch.manual_seed(args.seed)
    device = torch.device("cuda" if torch.cuda.is_available() and not args.no_cuda else "cpu")
    net, cfg = build_model(args, device)
    seqs = sorted({args.max_seq_length, max(8, args.max_seq_length // 2)})
    batches = [sample_inputs(cfg, b, s, device, args.seed + i)
               for i, (b, s) in enumerate([(args.batch_size, seqs[-1]), (1, seqs[0]), (max(1, args.batch_size // 2), seqs[-1])])]
    report = export_repository(net, batches, args.repository, args.model_name, args.format, args.version,
                               args.batch_size, args.instances, args.dynamic_batching_delay_us,
                               tuple(args.preferred_batch_sizes), args.tolerance)
    print(json.dumps(report))
    return report


if __name__ == "__main__":
    main()
