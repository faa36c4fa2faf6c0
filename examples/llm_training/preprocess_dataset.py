"""Tokenise a text corpus into the list-of-token-tensors file the trainers read with ``--dataset``.

Counterpart of the reference's examples/llm_training/preprocess_dataset.py (which tokenises
zai-org/LongAlign-10k from the hub).  This version works offline: the input is a local ``.jsonl`` file with a
``text`` (or ``messages``) field per line, or a plain text file with one document per line; the tokenizer is a
local Hugging Face tokenizer directory.

    python examples/llm_training/preprocess_dataset.py --input corpus.jsonl --tokenizer /path/to/tokenizer \
        --output data/corpus_tokens.pt --max-len 65536
"""
import argparse
import json

import torch


def documents(path):
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            if path.endswith(".jsonl"):
                rec = json.loads(line)
                if "messages" in rec:
                    yield "\n".join(m.get("content", "") for m in rec["messages"])
                else:
                    yield rec.get("text", "")
            else:
                yield line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--max-len", type=int, default=65536)
    args = ap.parse_args()
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(args.tokenizer)
    out = []
    for doc in documents(args.input):
        ids = tok(doc, add_special_tokens=True)["input_ids"][: args.max_len]
        if len(ids) >= 2:
            out.append(torch.tensor(ids, dtype=torch.int64))
    torch.save(out, args.output)
    lens = [int(t.numel()) for t in out]
    print(f"{len(out)} sequences, {sum(lens)} tokens, longest {max(lens) if lens else 0} -> {args.output}")


if __name__ == "__main__":
    main()
