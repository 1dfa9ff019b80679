#!/usr/bin/env python
"""Generate with any registered model folder (config.json + weights): the class is chosen by config.json.

    python examples/inflight/run.py --model_dir DIR --input_tokens prompts.csv --max_output_len 32 [--dtype bfloat16]
                                    [--top_k 1 --top_p 0 --temperature 1 --random_seed 0] [--max_step_tokens 512]

Models served in-flight (ragged batches: ``InflightSession``) take any number of prompts of any lengths; they queue for
state slots and cache pages, prompts are read in portions beside the running decodes.  A LLaMA engine folder (written by
examples/llama_quant/build.py) is run by ``GenerationSession`` as examples/llama_quant/run.py does."""
import argparse
import csv
import os
import sys
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--model_dir", required=True)
    p.add_argument("--input_tokens", required=True, help="CSV file: one prompt of token ids per line")
    p.add_argument("--max_output_len", type=int, required=True)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--max_seqs", type=int, default=8, help="state slots = sequences live at once")
    p.add_argument("--max_tokens", type=int, default=0, help="cache positions (default: room for max_seqs longest prompts)")
    p.add_argument("--max_step_tokens", type=int, default=512)
    p.add_argument("--top_k", type=int, default=1)
    p.add_argument("--top_p", type=float, default=0.0)
    p.add_argument("--temperature", type=float, default=1.0)
    p.add_argument("--random_seed", type=int, default=0)
    p.add_argument("--end_id", type=int, default=None)
    p.add_argument("--output_csv", default=None)
    a = p.parse_args()

    import torch
    from trtllm_llama_b200 import _lib, models
    from trtllm_llama_b200 import runtime as rt
    from trtllm_llama_b200.inflight import InflightSession
    from trtllm_llama_b200.layers import LayerStackModel

    with open(a.input_tokens) as f:
        prompts = [[int(x) for x in row] for row in csv.reader(f) if row]
    sc = rt.SamplingConfig(end_id=a.end_id, top_k=a.top_k, top_p=a.top_p, temperature=a.temperature, random_seed=a.random_seed)
    _lib.load_ragged_library(build=True)
    model = models.load_model(a.model_dir, dtype=a.dtype)
    t0 = time.time()
    if isinstance(model, LayerStackModel):
        longest = max(len(q) for q in prompts) + a.max_output_len
        sess = InflightSession(model, a.max_tokens or a.max_seqs * (longest + 64), a.max_seqs)
        outs = sess.generate(prompts, a.max_output_len, sc, a.max_step_tokens)
    else:
        mc, tensors = model
        sess = rt.GenerationSession(mc, tensors)
        S = max(len(q) for q in prompts)
        ids = torch.full((len(prompts), S), sc.pad_id, dtype=torch.int32)
        for i, q in enumerate(prompts):
            ids[i, :len(q)] = torch.tensor(q, dtype=torch.int32)
        sess.setup(len(prompts), S, a.max_output_len)
        outs = sess.decode(ids.pin_memory(), torch.tensor([len(q) for q in prompts], dtype=torch.int32), sc).tolist()
    torch.cuda.synchronize()
    dt = time.time() - t0
    for q, o in zip(prompts, outs):
        print(f"Input ids: {q}")
        print(f"Output ids: {o}")
    print(f"{sum(len(o) for o in outs)} tokens in {dt:.3f} s")
    if a.output_csv:
        with open(a.output_csv, "w") as f:
            csv.writer(f).writerows(outs)


if __name__ == "__main__":
    main()
