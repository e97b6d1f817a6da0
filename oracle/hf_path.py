"""The reference's PyTorch path, driven on CPU: Hugging Face `transformers.models.qwen3_5` modules in plain torch.

TEST INFRASTRUCTURE ONLY (see oracle/ops.py). open-jev-fast measures itself against exactly this path (its E2E_MODE=torch,
bench/e2e_bench.py:16-20, and tests/test_correct.py:31-113 use the Hugging Face modules as the oracle); it has no prefix
tree, so every candidate prompt is run as its own full sequence. The caller passes a `Qwen3_5TextModel` with the weights
under test; `upcast=True` computes in fp32 on the bf16-valued weights, which is the comparison target of the parity tests
(`upcast=False` keeps the bf16 arithmetic of the reference's own run and serves as the timed CPU baseline).
"""
import copy

import torch


def prepare(core, upcast=True):
    """A CPU copy of `core` ready for the oracle runs."""
    c = copy.deepcopy(core).to("cpu")
    c.eval()
    return c.float() if upcast else c


@torch.no_grad()
def candidate_hidden(core_cpu, seqs):
    """Final-norm hidden state of the last token of every candidate prompt: fp32 [S, H]."""
    out = []
    for s in seqs:
        ids = torch.tensor([list(s)], dtype=torch.long)
        out.append(core_cpu(input_ids=ids).last_hidden_state[0, -1].float())
    return torch.stack(out)


@torch.no_grad()
def all_hidden(core_cpu, seq):
    """Final-norm hidden state of every token of one sequence: fp32 [T, H]."""
    ids = torch.tensor([list(seq)], dtype=torch.long)
    return core_cpu(input_ids=ids).last_hidden_state[0].float()


def scores(hidden, head_w, head_b=None):
    """fp32 Linear on the gathered hidden states (src/server.py:37): [S, H] -> [S, A]."""
    y = hidden.float() @ head_w.float().cpu().t()
    return y if head_b is None else y + head_b.float().cpu()


@torch.no_grad()
def gdn_layer(layer, x, output_final_state=False):
    """One Qwen3_5GatedDeltaNet module on x [1, T, H] -> [1, T, H]."""
    return layer(hidden_states=x)


@torch.no_grad()
def time_layers(core_cpu, seqs, reps=1):
    """Seconds for one linear-attention decoder layer and one full-attention decoder layer (each including its MLP) over
    all candidate paths, for the extrapolated CPU baseline. Returns (t_linear, t_full)."""
    import time
    cfg = core_cpu.config
    types = list(cfg.layer_types)
    li, fi = types.index("linear_attention"), types.index("full_attention")
    res = []
    for idx in (li, fi):
        layer = core_cpu.layers[idx]
        best = float("inf")
        for _ in range(reps + 1):
            t0 = time.perf_counter()
            for s in seqs:
                T = len(s)
                x = torch.randn(1, T, cfg.hidden_size, dtype=next(layer.parameters()).dtype)
                pos = torch.arange(T)[None]
                pe = core_cpu.rotary_emb(x, pos)
                mask = torch.full((T, T), float("-inf"), dtype=x.dtype).triu(1)[None, None]
                layer(x, position_embeddings=pe, attention_mask=mask if idx == fi else None, position_ids=pos)
            best = min(best, time.perf_counter() - t0)
        res.append(best)
    return tuple(res)
