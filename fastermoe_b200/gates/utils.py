"""Capacity limiting shared by the balanced gates."""
import torch

from .. import fmoe_cuda as fmoe_native


def limit_by_capacity(topk_idx, num_expert, world_size, capacity):
    r"""Caps the number of tokens each expert accepts at ``capacity``.

    Intended behaviour of fmoe/gates/utils.py:9-26 (whose unpacking of
    ``count_by_gate`` / ``expert_exchange`` no longer matches those functions):
    count locally, exchange, let every expert grant its sources in ascending
    rank order up to ``capacity``, send the grants back, and set the local gate
    entries beyond each grant to -1 (lowest flat index kept first).

    ``capacity``: rows each local expert accepts, an int or an int tensor [num_expert].
    Returns ``(new_lec, new_gec, topk_idx)``.
    """
    with torch.no_grad():
        n_tot = num_expert * world_size
        if torch.is_tensor(capacity):     # one allowance per local expert
            cap = capacity.to(device=topk_idx.device, dtype=torch.int32).reshape(num_expert).clone()
        else:
            cap = torch.full((num_expert,), int(capacity), dtype=torch.int32, device=topk_idx.device)
        lec32 = torch.zeros(n_tot, dtype=torch.int32, device=topk_idx.device)
        fmoe_native.expert_count(topk_idx.reshape(-1).contiguous(), lec32)
        lec = lec32.long()
        if world_size > 1:
            _, _, gec = fmoe_native.expert_exchange(lec, num_expert, world_size)
        else:
            gec = lec
        new_gec = fmoe_native.limit_by_capacity(gec, cap, num_expert, world_size)
        if world_size > 1:
            # Sending the grants back is the same transpose as the count exchange.
            _, _, new_lec = fmoe_native.expert_exchange(new_gec, num_expert, world_size)
        else:
            new_lec = new_gec
        pruned = fmoe_native.prune_gate_by_capacity(topk_idx.contiguous(), new_lec.to(torch.int32),
                                                    num_expert, world_size)
    return new_lec, new_gec, pruned
