"""Stand-in for the FlashAttention-3 Python interface, which is Hopper-only (wgmma) and not in this image.

The reference record script imports ``flash_attn_func`` from this module name; here it maps onto
``torch.nn.functional.scaled_dot_product_attention`` with whatever SDPA backends the script itself enabled
(it turns on the flash backend only). Inputs and output are [batch, seq, heads, head_dim]."""
import torch.nn.functional as F


def flash_attn_func(q, k, v, causal=False, softmax_scale=None):
    out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal, scale=softmax_scale,
                                         enable_gqa=q.size(2) != k.size(2))
    return out.transpose(1, 2)
