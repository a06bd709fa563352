"""CPU reference of the expert-parallel regroup plan (TEST INFRASTRUCTURE).

The reference project has no expert parallelism (data parallelism only, ``train.py:944-949``; a sketch in
``aidocs/moe.md:940-997``), so there is nothing of the reference to restate here: this file states, in plain torch,
the layout contract that ``lmoe_ep_plan`` implements, and the tests check the kernel against it and the whole
exchange against the single-rank oracle."""
import torch


def regroup_tables(counts_all: torch.Tensor, rank: int):
    """counts_all[G, E] -> (recv_pos, row_src, pad_offsets, tile_expert, n_tiles) for `rank`.

    Receive order: source rank, then local expert.  Padded order: local expert, then source rank, each expert's
    segment rounded up to 128 rows."""
    G, E = counts_all.shape
    El = E // G
    cnt = counts_all[:, rank * El:(rank + 1) * El].long()            # [source, local expert]
    tot = cnt.sum(0)
    padded = (tot + 127) // 128 * 128
    pad_offsets = torch.cat([torch.zeros(1, dtype=torch.long), padded.cumsum(0)])
    n_recv = int(cnt.sum())
    recv_pos = torch.empty(n_recv, dtype=torch.long)
    row_src = torch.full((int(pad_offsets[-1]),), -1, dtype=torch.long)
    i = 0
    for s in range(G):
        for j in range(El):
            n = int(cnt[s, j])
            dst0 = int(pad_offsets[j] + cnt[:s, j].sum())
            recv_pos[i:i + n] = torch.arange(dst0, dst0 + n)
            row_src[dst0:dst0 + n] = torch.arange(i, i + n)
            i += n
    tile_expert = torch.repeat_interleave(torch.arange(El), padded // 128)
    return recv_pos, row_src, pad_offsets, tile_expert, int(pad_offsets[-1]) // 128
