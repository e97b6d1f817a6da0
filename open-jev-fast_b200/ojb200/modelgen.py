"""Random-init Qwen3.5-style hybrid backbones for tests and benchmarks (no checkpoint is downloaded).

The backbone object is Hugging Face's `Qwen3_5TextModel` — the module tree that open-jev-fast's FastQwen35 reads its weights
from (src/fastmodel.py:72-112) and whose plain-torch forward is "the reference's PyTorch path". Weights are drawn from a
generator keyed by (seed, parameter name), so the same values can be produced again on another device or in another
process without shipping a file.
"""
import zlib

import torch

# the fused Triton / causal-conv1d fast paths of transformers must stay off: the comparison path is the pure-torch one
# (what open-jev-fast's bench/e2e_bench.py:16-20 selects with E2E_MODE=torch)
import transformers.utils.import_utils as _iu

_iu.is_flash_linear_attention_available = lambda: False
_iu.is_causal_conv1d_available = lambda: False
try:
    import transformers.utils as _tu
    _tu.is_flash_linear_attention_available = _iu.is_flash_linear_attention_available
    _tu.is_causal_conv1d_available = _iu.is_causal_conv1d_available
except Exception:  # pragma: no cover
    pass

FULL = dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=64, num_attention_heads=24,
            num_key_value_heads=4, head_dim=256, linear_num_key_heads=16, linear_num_value_heads=32,
            linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4, vocab_size=4096)
SMALL = dict(hidden_size=256, intermediate_size=512, num_hidden_layers=8, num_attention_heads=4,
             num_key_value_heads=2, head_dim=128, linear_num_key_heads=2, linear_num_value_heads=4,
             linear_key_head_dim=128, linear_value_head_dim=128, linear_conv_kernel_dim=4, vocab_size=512)


def make_config(**over):
    """Qwen3_5TextConfig with full attention on every 4th layer; `over` overrides FULL (the 27B-scale dimensions the
    benchmark is quoted on: hidden 5120, MLP 17408, 64 layers, 24/4 attention heads of 256, GDN 16 key / 32 value heads of 128)."""
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5TextConfig
    d = dict(FULL)
    d.update(over)
    L = d["num_hidden_layers"]
    d.setdefault("layer_types", ["full_attention" if i % 4 == 3 else "linear_attention" for i in range(L)])
    d.setdefault("rms_norm_eps", 1e-6)
    d.setdefault("max_position_embeddings", 32768)
    cfg = Qwen3_5TextConfig(**d)
    cfg._attn_implementation = "eager"
    return cfg


def _gen(seed, name, device):
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) % (2 ** 63 - 1))
    return g


@torch.no_grad()
def fill_weights(core, seed=0, std=0.02, draw_on=None):
    """Overwrite every parameter of `core` in place from the (seed, name)-keyed generator.
    Linear / embedding / conv weights ~ N(0, std); RMSNorm weights ~ N(0, std) (they enter as 1 + w); the gated-norm weight
    ~ 1 + N(0, std); A_log = log U(0, 16) and dt_bias = 1 as Hugging Face initialises them. `draw_on` = device on which the
    random numbers are drawn ("cpu" gives identical values on every machine; None draws on the parameter's device)."""
    for name, p in core.named_parameters():
        dev = p.device if draw_on is None else torch.device(draw_on)
        g = _gen(seed, name, dev)
        if name.endswith("A_log"):
            v = torch.log(torch.rand(p.shape, generator=g, device=dev) * 16 + 1e-3)
        elif name.endswith("dt_bias"):
            v = torch.ones(p.shape, device=dev)
        elif name.endswith("linear_attn.norm.weight"):
            v = 1.0 + torch.randn(p.shape, generator=g, device=dev) * std
        else:
            v = torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) * std
        p.copy_(v.to(p.dtype))
    return core


def build_core(cfg, device="cuda", dtype=torch.bfloat16, seed=0, std=0.02, draw_on=None):
    """Hugging Face Qwen3_5TextModel with seeded weights, created directly on `device` in `dtype`."""
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5TextModel
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        with torch.device(device):
            core = Qwen3_5TextModel(cfg)
    finally:
        torch.set_default_dtype(old)
    core.eval()
    fill_weights(core, seed, std, draw_on)
    return core


def make_head(H, A=1, seed=0, device="cuda"):
    """Scoring head: fp32 Linear(H -> A) on the last-token hidden state. A = 1 is the scalar head open-jev-fast applies
    (src/server.py:37; the module itself lives in the un-vendored `jev` package); A > 1 reads a small answer vocabulary."""
    g = torch.Generator().manual_seed(seed * 7919 + 17)
    W = (torch.randn(A, H, generator=g) * H ** -0.5).to(device)
    b = (torch.randn(A, generator=g) * 0.1).to(device)
    return W, b
