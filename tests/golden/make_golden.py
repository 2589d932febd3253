"""Run jason-fxz/mini-sglang's own Qwen3 model code on the CPU in float32 on the tiny random
models of tests/tiny_models.py and store its logits as goldens for tests/plain_qwen3.py.

    python tests/golden/make_golden.py /path/to/mini-sglang-checkout

What it does: imports `mini_sglang.models.qwen3.Qwen3ForCausalLM` from the checkout, builds
it from a SimpleNamespace configuration, loads the tiny weights through the model's own
`load_weights`, and drives it with hand-built EXTEND batches over the project's
`TorchNativeAttnBackend` (page size 1, CPU tensors).  The reference returns only the last
row of a request, so the sequence is replayed once per prefix length.  Written to
tests/golden/ref_<name>.pt: {"tokens", "logits" [S, vocab] float32}.  The stored files are
what tests/test_plain.py compares the plain implementation with; this script is only
needed to regenerate them.
"""

from __future__ import annotations

import os
import sys
import types

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from tiny_models import CONFIGS, make_weights, random_tokens  # noqa: E402

SEQ_LEN = {"A": 13, "B": 23, "C": 11}
SEEDS = {"A": 0, "B": 1, "C": 2}


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    import torch.distributed as dist

    dist.init_process_group(backend="gloo", rank=0, world_size=1)
    from mini_sglang.layers.attn.torch_attn_backend import TorchNativeAttnBackend
    from mini_sglang.managers.batch_info import BatchInfo, ForwardMode
    from mini_sglang.mem_cache.req2token import ReqToTokenPool
    from mini_sglang.mem_cache.token2kv import MHAKVPool
    from mini_sglang.models.qwen3 import Qwen3ForCausalLM

    torch.set_default_dtype(torch.float32)
    for name, cfg in CONFIGS.items():
        ns = types.SimpleNamespace(**{k: v for k, v in cfg.items()})
        model = Qwen3ForCausalLM(ns)
        weights = make_weights(cfg, SEEDS[name])
        model.load_weights([(k, v.to(torch.float32)) for k, v in weights.items()])
        d = cfg["head_dim"]
        S = SEQ_LEN[name]
        toks = random_tokens(S, cfg["vocab_size"], 100 + SEEDS[name])
        r2t = ReqToTokenPool(size=2, max_tokens=64, page_size=1, device="cpu")
        kv = MHAKVPool(size=64, page_size=1, dtype=torch.float32, head_num=cfg["num_key_value_heads"],
                       head_dim=d, layer_num=cfg["num_hidden_layers"], device="cpu")
        backend = TorchNativeAttnBackend(types.SimpleNamespace(device="cpu", req_to_token_pool=r2t, kv_cache_pool=kv))
        rows = []
        with torch.inference_mode():
            for n in range(1, S + 1):
                loc = [1 + i for i in range(n)]
                r2t.req_to_token[0, :n] = torch.tensor(loc, dtype=torch.int32)
                b = BatchInfo(forward_mode=ForwardMode.EXTEND, reqs=[None], device="cpu",
                              input_ids=torch.tensor(toks[:n], dtype=torch.int32),
                              positions=torch.arange(n, dtype=torch.int32),
                              input_seq_lens=torch.tensor([n], dtype=torch.int32),
                              seq_lens=torch.tensor([n], dtype=torch.int32),
                              prefix_seq_lens=torch.tensor([0], dtype=torch.int32),
                              out_cache_loc=torch.tensor(loc, dtype=torch.int32),
                              req_pool_indices=torch.tensor([0], dtype=torch.int32),
                              req_to_token_pool=r2t, kv_cache_pool=kv, attn_backend=backend)
                rows.append(model.forward(b.input_ids, b.positions, b).next_token_logits[0].clone())
        out = {"tokens": toks, "logits": torch.stack(rows).to(torch.float32)}
        torch.save(out, os.path.join(HERE, f"ref_{name}.pt"))
        print(name, "stored", tuple(out["logits"].shape))
    dist.destroy_process_group()


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/mini-sglang-checkout")
    main(sys.argv[1])
