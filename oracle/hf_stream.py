"""The reference's PyTorch path run one decoder layer at a time, for models too large to hold a second (fp32) copy of.

TEST INFRASTRUCTURE ONLY (see oracle/ops.py). Same arithmetic as oracle/hf_path.py — the Hugging Face `qwen3_5` modules in
plain torch, one full sequence per candidate prompt (open-jev-fast's E2E_MODE=torch, bench/e2e_bench.py:16-20; its
tests/test_correct.py:31-113 use these modules as the oracle) — but the 64-layer, 27B-parameter model of the benchmark does
not fit a GPU twice in fp32, so every decoder layer is copied to the comparison precision, applied to all candidates, and
released before the next one. tests/test_oracle_hf.py pins this streamed run against the whole-model forward of
oracle/hf_path.py; tests/test_full_model_gpu.py cross-checks a GPU run of one layer of each type against the CPU run.

Arms (`mode`):
  "fp32"     every layer upcast to fp32 (weights keep their bf16 values): the comparison target of the parity tests
  "bf16"     the layers as they are — what the reference's own PyTorch path computes when it runs the model in bf16
  "operands" fp32 arithmetic, except that the input of every nn.Linear is rounded to bf16 first: the least error any
             implementation whose projections take bf16 operands can have (a floor, not an implementation)
"""
import copy

import torch


def _round_linear_inputs(layer):
    def pre(_m, args):
        return (args[0].to(torch.bfloat16).to(args[0].dtype),) + tuple(args[1:])
    for m in layer.modules():
        if isinstance(m, torch.nn.Linear):
            m.register_forward_pre_hook(pre)


def _layer_copy(layer, mode):
    if mode == "bf16":
        return layer
    c = copy.deepcopy(layer).float()
    if mode == "operands":
        _round_linear_inputs(c)
    return c


@torch.no_grad()
def candidate_hidden(core, seqs, mode="fp32", n_layers=None, all_rows=False):
    """Final-norm hidden state of the last token of every candidate prompt, fp32 [S, H] (all_rows=True: list of [T_s, H]).
    `core` is a Hugging Face Qwen3_5TextModel holding the (bf16-valued) weights under test on any device; the run happens
    on that device. n_layers truncates the model (the final norm is applied after layer n_layers - 1)."""
    torch.set_float32_matmul_precision("highest")
    cfg = core.config
    dev = core.embed_tokens.weight.device
    dt = torch.bfloat16 if mode == "bf16" else torch.float32
    xs, pes, masks, poss = [], [], [], []
    for s in seqs:
        ids = torch.tensor([list(s)], dtype=torch.long, device=dev)
        x = core.embed_tokens(ids).to(dt)
        T = x.shape[1]
        pos = torch.arange(T, device=dev)
        pe = core.rotary_emb(x, pos.view(1, 1, T).expand(3, 1, T))
        mask = torch.full((T, T), torch.finfo(dt).min, dtype=dt, device=dev).triu(1)[None, None]
        xs.append(x), pes.append(pe), masks.append(mask), poss.append(pos[None])
    types = list(cfg.layer_types)
    nl = len(core.layers) if n_layers is None else n_layers
    for i in range(nl):
        L = _layer_copy(core.layers[i], mode)
        full = types[i] == "full_attention"
        for j in range(len(xs)):
            xs[j] = L(xs[j], position_embeddings=pes[j], attention_mask=masks[j] if full else None, position_ids=poss[j])
        del L
    norm = core.norm if mode == "bf16" else copy.deepcopy(core.norm).float()
    if all_rows:
        return [norm(x)[0].float() for x in xs]
    return torch.stack([norm(x)[0, -1].float() for x in xs])


@torch.no_grad()
def one_layer(layer, cfg, rotary, x, device, mode="fp32"):
    """One decoder layer (copied to `device` in the arm's precision) on x [1, T, H] -> [1, T, H] fp32 on the CPU. Used to
    cross-check a GPU run of the oracle against the CPU run of the same layer."""
    torch.set_float32_matmul_precision("highest")
    dt = torch.bfloat16 if mode == "bf16" else torch.float32
    L = copy.deepcopy(layer).to(device)
    L = L.float() if mode != "bf16" else L
    if mode == "operands":
        _round_linear_inputs(L)
    x = x.to(device=device, dtype=dt)
    T = x.shape[1]
    pos = torch.arange(T, device=device)
    pe = copy.deepcopy(rotary).to(device)(x, pos.view(1, 1, T).expand(3, 1, T))
    mask = torch.full((T, T), torch.finfo(dt).min, dtype=dt, device=device).triu(1)[None, None]
    full = getattr(L, "layer_type", None) == "full_attention"
    return L(x, position_embeddings=pe, attention_mask=mask if full else None, position_ids=pos[None]).float().cpu()
