"""Per-token hidden states of chosen BERT layers for a text file, one JSON object per line.

Input lines are ``sentence`` or ``sentence a ||| sentence b`` (the convention of the reference's
``examples/BertPretraining/extract_features.py:168-189``); the output mirrors its JSON
(``:262-286``): ``{"linex_index": i, "features": [{"token": t, "layers": [{"index": -1,
"values": [...]}, ...]}, ...]}``.

    python examples/bert_pretraining/extract_features.py --input_file text.txt --output_file out.jsonl \
        --vocab_file vocab.txt --bert_model base [--init_checkpoint ckpt.pt] --layers -1,-2
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from conef_b200 import models  # noqa: E402
from conef_b200.data.glue import encode_pair  # noqa: E402
from conef_b200.data.tokenization import BertTokenizer  # noqa: E402


def read_examples(path):
    out = []
    with open(path, encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            a, sep, b = line.partition("|||")
            out.append((a.strip(), b.strip() if sep else None))
    return out


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--input_file", required=True)
    p.add_argument("--output_file", required=True)
    p.add_argument("--vocab_file", required=True)
    p.add_argument("--bert_model", default="base", choices=["large", "base", "tiny"])
    p.add_argument("--config_file", default=None)
    p.add_argument("--init_checkpoint", default=None, help="checkpoint with a 'model' state dict")
    p.add_argument("--do_lower_case", action="store_true", default=True)
    p.add_argument("--layers", default="-1,-2,-3,-4")
    p.add_argument("--max_seq_length", type=int, default=128)
    p.add_argument("--batch_size", type=int, default=32)
    p.add_argument("--no_cuda", action="store_true")
    args = p.parse_args()

    device = torch.device("cuda" if torch.cuda.is_available() and not args.no_cuda else "cpu")
    tok = BertTokenizer(args.vocab_file, do_lower_case=args.do_lower_case)
    if args.config_file:
        cfg = models.BertConfig.from_json_file(args.config_file)
    elif args.bert_model == "large":
        cfg = models.BertConfig.large()
    elif args.bert_model == "base":
        cfg = models.BertConfig.base()
    else:
        cfg = models.BertConfig(max(len(tok.vocab), 8), hidden_size=128, num_hidden_layers=2,
                                num_attention_heads=4, intermediate_size=512)
    cfg.output_all_encoded_layers = True
    net = models.BertModel(cfg)
    if args.init_checkpoint:
        sd = torch.load(args.init_checkpoint, map_location="cpu")
        sd = sd.get("model", sd)
        sd = {k.split("bert.", 1)[-1]: v for k, v in sd.items() if "bert." in k or not k.startswith("cls.")}
        missing, unexpected = net.load_state_dict(sd, strict=False)
        print(f"loaded {args.init_checkpoint}: {len(missing)} missing, {len(unexpected)} unexpected keys")
    net = net.to(device).eval()
    layer_idx = [int(x) for x in args.layers.split(",")]
    examples = read_examples(args.input_file)
    encoded = [encode_pair(tok, a, b, args.max_seq_length) for a, b in examples]

    with open(args.output_file, "w", encoding="utf-8") as out, torch.no_grad():
        for lo in range(0, len(encoded), args.batch_size):
            chunk = encoded[lo : lo + args.batch_size]
            ids = torch.tensor([c[1] for c in chunk], device=device)
            mask = torch.tensor([c[2] for c in chunk], device=device)
            seg = torch.tensor([c[3] for c in chunk], device=device)
            layers, _ = net(ids, seg, mask)
            for k, (tokens, *_rest) in enumerate(chunk):
                feats = []
                for t, token in enumerate(tokens):
                    feats.append({"token": token, "layers": [
                        {"index": li, "values": [round(float(x), 6) for x in layers[li][k, t].float().cpu()]}
                        for li in layer_idx]})
                out.write(json.dumps({"linex_index": lo + k, "features": feats}) + "\n")
    print(f"{len(encoded)} lines -> {args.output_file}")


if __name__ == "__main__":
    main()
