"""CPU sampling path (torch RNG); same contract as the CUDA kernel, different random stream."""

from __future__ import annotations

import torch

from slime_b200.ops.reference import topp_topk_keep_mask


def sample_reference(logits, temperature, top_k=None, top_p=None, min_p=None, seeds=None, positions=None, kept_cap=0):
    B, V = logits.shape
    token = torch.empty(B, dtype=torch.int32)
    logprob = torch.empty(B, dtype=torch.float32)
    kept_ids = torch.zeros(B, kept_cap, dtype=torch.int32) if kept_cap > 0 else None
    kept_count = torch.zeros(B, dtype=torch.int32) if kept_cap > 0 else None
    for b in range(B):
        t = float(temperature[b])
        z = logits[b].float()
        if t <= 0:
            tok = int(z.argmax())
            token[b] = tok
            logprob[b] = torch.log_softmax(z, -1)[tok]
            if kept_cap > 0:
                kept_ids[b, 0], kept_count[b] = tok, 1
            continue
        probs = torch.softmax(z / t, -1)
        k = int(top_k[b]) if top_k is not None else 0
        p = float(top_p[b]) if top_p is not None else 1.0
        mp = float(min_p[b]) if min_p is not None else 0.0
        filtered = (0 < k < V) or p < 1.0 or mp > 0
        keep = topp_topk_keep_mask(probs, k, p, mp) if filtered else torch.ones(V, dtype=torch.bool)
        masked = torch.where(keep, probs, torch.zeros_like(probs))
        gen = torch.Generator()
        seed = int(seeds[b]) if seeds is not None else 0x1234 + b
        pos = int(positions[b]) if positions is not None else 0
        gen.manual_seed((seed * 1000003 + pos) % (2**63))
        tok = int(torch.multinomial(masked / masked.sum(), 1, generator=gen))
        token[b] = tok
        logprob[b] = torch.log(probs[tok] / masked.sum())
        if kept_cap > 0 and filtered:
            ids = torch.nonzero(keep, as_tuple=True)[0][:kept_cap].to(torch.int32)
            kept_ids[b, : ids.numel()] = ids
            kept_count[b] = ids.numel()
    return token, logprob, kept_ids, kept_count
