"""The reference's CPU path for a decode / verify / prompt-chunk row, restated with the same torch ops (TEST AND
BASELINE INFRASTRUCTURE ONLY; the product never imports it): gather the row's pages through its block table
(index_select), dequantise to the pool's compute dtype (code * scale in FP32, then bf16), and torch's scaled dot
product attention with GQA.
ref: inference/attention-state/code/pages.py:455-477 (KVPool.gather) and
     inference/attention-state/code/device_attention.py:1148-1166 (_gathered).
The per-(page, kv head) FP8 kind has no reference code: its scales [pages][kv_heads] are broadcast over the page's
positions, the row rule otherwise."""
import math

import torch


def gather(codes, scales, table, count, page, kind, multiplier=1.0, compute=torch.bfloat16):
    """codes [pages][page][hkv][dim] (uint8 views of E4M3 for the FP8 kinds) -> [count][hkv][dim] in `compute`."""
    needed = math.ceil(count / page)
    index = table[:needed].long()
    rows = codes.index_select(0, index)
    n = needed * page
    hkv, dim = rows.shape[-2], rows.shape[-1]
    if kind in ("bf16", "fp16", "fp32"):
        return rows.reshape(n, hkv, dim)[:count].to(compute)
    values = (rows.view(torch.float8_e4m3fn) if kind != "int8" else rows).float().reshape(n, hkv, dim)[:count]
    if kind == "fp8":
        return (values * multiplier).to(compute)
    picked = scales.index_select(0, index)
    if kind == "fp8:page":
        picked = picked[:, None, :].expand(needed, page, hkv)
    return (values * picked.reshape(n, hkv)[:count, :, None]).to(compute)


def attend_row(q, keys, values, position, scale):
    """q [count][hq][d] at positions position.. over gathered keys/values [position + count][hkv][d]: SDPA with the
    offset causal mask the reference builds (none for one token)."""
    count, heads = q.shape[0], q.shape[1]
    qq = q.transpose(0, 1).unsqueeze(0).to(keys.dtype)
    k, v = keys.transpose(0, 1).unsqueeze(0), values.transpose(0, 1).unsqueeze(0)
    mask, causal = None, count > 1 and position == 0
    if count > 1 and position > 0:
        seen = torch.arange(position + count)
        mask = seen[None, :] <= (position + torch.arange(count))[:, None]
    found = torch.nn.functional.scaled_dot_product_attention(qq, k, v, attn_mask=mask, is_causal=causal, scale=scale,
                                                             enable_gqa=heads != keys.shape[1])
    return found[0].transpose(0, 1)


def decode_step(q, k_codes, v_codes, k_scales, v_scales, tables, firsts, counts, page, kind, scale=None,
                multipliers=(1.0, 1.0)):
    """Rows of counts[r] tokens at positions firsts[r].. (CPU tensors) -> out [tokens][hq][dv] in q's dtype."""
    scale = scale if scale is not None else q.shape[-1] ** -0.5
    out = torch.empty(q.shape[0], q.shape[1], v_codes.shape[-1], dtype=q.dtype)
    at = 0
    for r, (first, count) in enumerate(zip(firsts, counts)):
        n = first + count
        keys = gather(k_codes, k_scales, tables[r], n, page, kind, multipliers[0])
        values = gather(v_codes, v_scales, tables[r], n, page, kind, multipliers[1])
        out[at:at + count] = attend_row(q[at:at + count], keys, values, first, scale).to(out.dtype)
        at += count
    return out
