"""Question answering against an exported model: through a Triton server, or in-process from the
same model repository.

Counterpart of the reference's ``examples/BertPretraining/triton/client.py`` (one question and
context to the server, answer text back, ``:60-170``), ``triton/run_squad_client.py`` (a SQuAD
file through the server, predictions written as JSON, ``:120-280``) and ``triton/run_perf_client.sh``
(sequences per second at a batch size, the metric of the reference's only published table).

Two back ends with one interface, ``infer([ids, segments, mask]) -> [start_logits, end_logits]``:

* ``--triton_url host:port`` sends the request with ``tritonclient.http`` (needed only for this mode);
* ``--local_repository DIR`` loads ``DIR/<model_name>/<version>/model.pt`` with ``torch.jit.load`` and
  splits requests at the ``max_batch_size`` of ``config.pbtxt``, as the server's batcher would.

    python examples/bert_pretraining/deploy/client.py --local_repository /models --model_name bert_qa \
        --vocab_file vocab.txt --question "Who wrote it?" --context "It was written by Ada."
    python examples/bert_pretraining/deploy/client.py --local_repository /models --squad_file dev-v1.1.json \
        --vocab_file vocab.txt --output_file predictions.json
    python examples/bert_pretraining/deploy/client.py --local_repository /models --perf --batch_size 8
"""
import argparse
import json
import os
import re
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", ".."))
sys.path.insert(0, os.path.join(HERE, ".."))

from inference import best_spans, build_features  # noqa: E402
from conef_b200.data.squad import squad_scores  # noqa: E402,F401
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402


def read_config(path):
    """The few fields of ``config.pbtxt`` a client needs: ``max_batch_size`` and the tensor names."""
    text = open(path).read()
    m = re.search(r"max_batch_size:\s*(\d+)", text)
    names = re.findall(r'name:\s*"((?:input|output)__\d+)"', text)
    return {"max_batch_size": int(m.group(1)) if m else 0,
            "inputs": [n for n in names if n.startswith("input")],
            "outputs": [n for n in names if n.startswith("output")]}


class LocalBackend:
    """Runs the exported TorchScript file of a model repository in this process."""

    def __init__(self, repository, model_name, version=1, device=None):
        import torch
        self.torch = torch
        model_dir = os.path.join(repository, model_name)
        self.config = read_config(os.path.join(model_dir, "config.pbtxt"))
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.model = torch.jit.load(os.path.join(model_dir, str(version), "model.pt"), map_location=self.device)
        self.model.eval()

    def infer(self, arrays):
        torch = self.torch
        n = arrays[0].shape[0]
        step = self.config["max_batch_size"] or n
        outs = None
        with torch.no_grad():
            for lo in range(0, n, step):
                part = [torch.from_numpy(np.ascontiguousarray(a[lo:lo + step])).to(self.device) for a in arrays]
                res = self.model(*part)
                res = [res] if torch.is_tensor(res) else list(res)
                res = [r.float().cpu().numpy() for r in res]
                outs = res if outs is None else [np.concatenate([o, r]) for o, r in zip(outs, res)]
        return outs


class TritonBackend:
    """Sends requests to a running Triton Inference Server over HTTP."""

    def __init__(self, url, model_name, version=1):
        try:
            import tritonclient.http as http
        except ImportError as e:
            raise RuntimeError("--triton_url needs the tritonclient package; use --local_repository without it") from e
        self.http = http
        self.client = http.InferenceServerClient(url=url)
        self.model_name, self.version = model_name, str(version)
        cfg = self.client.get_model_config(model_name, self.version)
        self.config = {"max_batch_size": int(cfg.get("max_batch_size", 0)),
                       "inputs": [i["name"] for i in cfg["input"]], "outputs": [o["name"] for o in cfg["output"]]}

    def infer(self, arrays):
        http = self.http
        n = arrays[0].shape[0]
        step = self.config["max_batch_size"] or n
        outs = None
        for lo in range(0, n, step):
            ins = []
            for name, a in zip(self.config["inputs"], arrays):
                part = np.ascontiguousarray(a[lo:lo + step])
                inp = http.InferInput(name, list(part.shape), "INT64")
                inp.set_data_from_numpy(part)
                ins.append(inp)
            req = [http.InferRequestedOutput(o) for o in self.config["outputs"]]
            res = self.client.infer(self.model_name, ins, model_version=self.version, outputs=req)
            res = [res.as_numpy(o).astype(np.float32) for o in self.config["outputs"]]
            outs = res if outs is None else [np.concatenate([o, r]) for o, r in zip(outs, res)]
        return outs


def answer_batch(backend, tokenizer, pairs, max_seq_length=384, max_query_length=64, n_best_size=1,
                 max_answer_length=30, with_negative=False, null_score_diff_threshold=0.0):
    """Best spans for ``[(question, context), ...]``: one request for all pairs."""
    feats = [build_features(q, c, tokenizer, max_seq_length, max_query_length) for q, c in pairs]
    ids = np.asarray([f[0] for f in feats], dtype=np.int64)
    mask = np.asarray([f[1] for f in feats], dtype=np.int64)
    seg = np.asarray([f[2] for f in feats], dtype=np.int64)
    start, end = backend.infer([ids, seg, mask])
    out = []
    for i, f in enumerate(feats):
        n = len(f[3])
        out.append(best_spans(start[i, :n].tolist(), end[i, :n].tolist(), f[4], f[5], n_best_size,
                              max_answer_length, with_negative, null_score_diff_threshold))
    return out


def read_squad(path):
    """``[(id, question, context)]`` from a SQuAD v1.1 / v2.0 JSON file."""
    rows = []
    for article in json.load(open(path))["data"]:
        for para in article["paragraphs"]:
            for qa in para["qas"]:
                rows.append((qa["id"], qa["question"], para["context"]))
    return rows


def throughput(backend, batch_size, seq_length, iters=20, warmup=3, vocab=1000, seed=0):
    """Sequences per second of back-to-back requests of one size (wall clock around the requests: what
    a client of the served model sees)."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, (batch_size, seq_length), dtype=np.int64)
    seg = np.zeros_like(ids)
    mask = np.ones_like(ids)
    for _ in range(warmup):
        backend.infer([ids, seg, mask])
    t0 = time.perf_counter()
    for _ in range(iters):
        backend.infer([ids, seg, mask])
    dt = time.perf_counter() - t0
    return {"batch_size": batch_size, "seq_length": seq_length, "iters": iters,
            "seq_per_s": batch_size * iters / dt, "ms_per_request": 1e3 * dt / iters}


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--triton_url", default=None, help="host:port of a running server")
    p.add_argument("--local_repository", default=None, help="model repository to load in-process")
    p.add_argument("--model_name", default="bert_qa")
    p.add_argument("--model_version", type=int, default=1)
    p.add_argument("--vocab_file", default=None)
    p.add_argument("--do_lower_case", action="store_true", default=True)
    p.add_argument("--question", default=None)
    p.add_argument("--context", default=None)
    p.add_argument("--squad_file", default=None, help="SQuAD JSON; predictions go to --output_file")
    p.add_argument("--output_file", default="predictions.json")
    p.add_argument("--evaluate", action="store_true", help="score the predictions against the file's gold answers")
    p.add_argument("--batch_size", type=int, default=8)
    p.add_argument("--max_seq_length", type=int, default=384)
    p.add_argument("--max_query_length", type=int, default=64)
    p.add_argument("--n_best_size", type=int, default=1)
    p.add_argument("--max_answer_length", type=int, default=30)
    p.add_argument("--version_2_with_negative", action="store_true")
    p.add_argument("--null_score_diff_threshold", type=float, default=0.0)
    p.add_argument("--perf", action="store_true", help="measure sequences per second of random requests")
    p.add_argument("--perf_iters", type=int, default=20)
    p.add_argument("--perf_vocab", type=int, default=1000, help="random token ids are drawn below this")
    p.add_argument("--device", default=None, help="device of the in-process back end")
    args = p.parse_args(argv)
    if (args.triton_url is None) == (args.local_repository is None):
        p.error("give exactly one of --triton_url and --local_repository")
    backend = (TritonBackend(args.triton_url, args.model_name, args.model_version) if args.triton_url
               else LocalBackend(args.local_repository, args.model_name, args.model_version, args.device))
    if args.perf:
        res = throughput(backend, args.batch_size, args.max_seq_length, args.perf_iters, vocab=args.perf_vocab)
        print(json.dumps(res))
        return res
    if not args.vocab_file:
        p.error("--vocab_file is needed to answer questions")
    tok = BertTokenizer(args.vocab_file, do_lower_case=args.do_lower_case)
    kw = dict(max_seq_length=args.max_seq_length, max_query_length=args.max_query_length,
              n_best_size=args.n_best_size, max_answer_length=args.max_answer_length,
              with_negative=args.version_2_with_negative, null_score_diff_threshold=args.null_score_diff_threshold)
    if args.squad_file:
        rows = read_squad(args.squad_file)
        preds = {}
        for lo in range(0, len(rows), args.batch_size):
            chunk = rows[lo:lo + args.batch_size]
            for (qid, _, _), spans in zip(chunk, answer_batch(backend, tok, [(q, c) for _, q, c in chunk], **kw)):
                preds[qid] = spans[0]["text"]
        with open(args.output_file, "w") as f:
            json.dump(preds, f, indent=1)
        summary = {"questions": len(rows), "output_file": args.output_file}
        if args.evaluate:
            summary.update(squad_scores(preds, args.squad_file))
        print(json.dumps(summary))
        return preds
    if args.question is None or args.context is None:
        p.error("give --question and --context, --squad_file, or --perf")
    spans = answer_batch(backend, tok, [(args.question, args.context)], **kw)[0]
    res = {"question": args.question, "answers": spans}
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
