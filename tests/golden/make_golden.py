"""Makes ``tests/golden/reference_logits.pt``: logits of the reference's own model code on the CPU.

Run once, by hand, where the reference project is checked out::

    python tests/golden/make_golden.py /path/to/distie

It imports the reference's ``Qwen2CausalLM`` (worker/src/inference/qwen2/model.py:
293-314; the file needs torch only), builds it from the two tiny configurations of
``tests/helpers.py``, loads the seeded random weights of ``plain_qwen2.random_weights``
(checkpoint names minus the ``model.`` prefix, model.py:386-400), runs its dense
``forward`` and its paged ``forward_batch`` on a few sequences and stores the
float32 logits.  ``tests/test_plain.py`` compares the plain implementation with
the stored logits, so the oracle of all other tests is anchored in the
reference's own arithmetic without the reference being needed at test time.
"""

from __future__ import annotations

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

import helpers  # noqa: E402
import plain_qwen2 as plain  # noqa: E402


def main(reference_root: str) -> None:
    sys.path.insert(0, os.path.join(reference_root, "worker", "src"))
    from inference.kv_cache import KvShape, PagedKvCache
    from inference.qwen2.model import Qwen2CausalLM, Qwen2Dims
    from inference.qwen2.paged_attn import BatchSeq, build_batch

    out = {}
    for name in ("A", "B"):
        cfg, page, weights = helpers.tiny(name)
        dims = Qwen2Dims(
            vocab_size=cfg["vocab_size"], hidden_size=cfg["hidden_size"], intermediate_size=cfg["intermediate_size"],
            num_hidden_layers=cfg["num_hidden_layers"], num_attention_heads=cfg["num_attention_heads"],
            num_key_value_heads=cfg["num_key_value_heads"], head_dim=plain.head_dim_of(cfg),
            rms_norm_eps=cfg["rms_norm_eps"], rope_theta=cfg["rope_theta"], tie_word_embeddings=cfg["tie_word_embeddings"],
        )
        model = Qwen2CausalLM(dims).eval()
        state = {(k[len("model."):] if k.startswith("model.") else k): v for k, v in weights.items()}
        if cfg["tie_word_embeddings"]:
            state["lm_head.weight"] = state["embed_tokens.weight"]
        model.load_state_dict(state)
        ids = helpers.random_ids(cfg["vocab_size"], 45, 123)
        with torch.inference_mode():
            dense = model(torch.tensor([ids]))[0].float()
            # The reference's own paged, batched path: 29 tokens, then 16 more beside a second request.
            cache = PagedKvCache(KvShape(dims.num_hidden_layers, dims.num_key_value_heads, dims.head_dim), 16, "cpu", torch.float32, page)
            meta = build_batch([BatchSeq(tuple(range(8)), 0, 29)], cache, "cpu")
            model.forward_batch(torch.tensor(ids[:29]), cache, meta)
            other = helpers.random_ids(cfg["vocab_size"], 9, 7)
            meta = build_batch([BatchSeq(tuple(range(8)), 29, 16), BatchSeq(tuple(range(8, 12)), 0, 9)], cache, "cpu")
            paged_last = model.forward_batch(torch.tensor(ids[29:] + other), cache, meta)[0].float()
        out[name] = {"ids": ids, "dense": dense.clone(), "paged_last": paged_last.clone()}
        print(name, "dense", tuple(dense.shape), "paged-vs-dense", float((paged_last - dense[-1]).abs().max()))
    torch.save(out, os.path.join(HERE, "reference_logits.pt"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <checkout of the reference project>")
    main(sys.argv[1])
