"""Text generation with a Llama-architecture model (reference: examples/llama/main.go, generate.go).

    python examples/llama_generate.py                          # tiny random model, byte tokenizer
    python examples/llama_generate.py --model m.mim --prompt "Once upon"   # a .mim file with tokenizer metadata
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(model_path=None, prompt="hello", n=16, temperature=0.8, top_k=40, top_p=0.95, seed=0, log=print):
    from mimir_b200 import llm, nn
    if model_path:
        model = llm.Model.load(model_path)
        tok = llm.tokenizer_from_metadata(model.tokenizer_metadata)
    else:
        nn.manual_seed(seed)
        tokens = ["<unk>", "<s>", "</s>"] + [f"<0x{b:02X}>" for b in range(256)]
        tok = llm.SentencePiece(tokens, types=[2, 3, 3] + [6] * 256, bos=1, eos=2, add_space_prefix=False)
        model = llm.Model(llm.Config(vocab=len(tokens), context=64, embed=32, hidden=64, layers=2, heads=4, kv_heads=2,
                                     head_dim=8, rope_dim=8))
    ids = tok.encode(prompt)
    sampler = llm.Sampler(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed)
    out = llm.generate(model, ids, n, sampler, stop=(tok.eos,) if tok.eos is not None else ())
    text = tok.decode(out)
    log(prompt + text)
    return out, text


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model")
    ap.add_argument("--prompt", default="hello")
    ap.add_argument("-n", type=int, default=16)
    a = ap.parse_args()
    main(a.model, a.prompt, a.n)
