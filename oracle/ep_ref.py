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


def dedup_send_tables(sel: torch.Tensor, weights: torch.Tensor, counts_all: torch.Tensor, rank: int):
    """What one source rank writes in the de-duplicated exchange (the contract of ``lmoe_epd_send``).

    sel[T, K] (global expert ids), weights[T, K], counts_all[G, E].  Returns, per destination rank g, a dict with
      tokens   [n]        the tokens of this rank that own at least one expert of g (their staging slots are rank*stride + t)
      mask     [T]        bit k set: slot k of token t belongs to g
      slots    [T, K]     padded row of slot k in g's layout, -1 where the bit is clear
      meta_rows / meta_tok / meta_w   for every routed row sent to g: its padded row there, its token, its weight
    Padded row of a routed row of expert e = (g, j), the q-th row of this rank for e in canonical order:
      pad_off_g[j] + sum_{s < rank} counts_all[s][e] + q."""
    G, E = counts_all.shape
    El = E // G
    T, K = sel.shape
    flat = sel.reshape(-1)
    perm = torch.argsort(flat, stable=True)                       # canonical order (expert, then flat index)
    own_counts = torch.bincount(flat, minlength=E)
    offsets = torch.cat([torch.zeros(1, dtype=torch.long), own_counts.cumsum(0)])
    pos = torch.empty_like(perm)
    pos[perm] = torch.arange(perm.numel())
    tot = counts_all.long().sum(0)
    padded = (tot + 127) // 128 * 128
    out = []
    for g in range(G):
        pad_off = torch.cat([torch.zeros(1, dtype=torch.long), padded[g * El:(g + 1) * El].cumsum(0)])
        mine = (sel // El) == g                                     # [T, K]
        e = sel.clamp(min=0)
        before = counts_all[:rank].long().sum(0)                    # rows of lower ranks per expert
        q = pos.view(T, K) - offsets[e]
        drow = pad_off[(e - g * El).clamp(0, El - 1)] + before[e] + q
        slots = torch.where(mine, drow, torch.full_like(drow, -1))
        mask = (mine.long() << torch.arange(K)).sum(1)
        out.append(dict(tokens=mine.any(1).nonzero().flatten(), mask=mask, slots=slots,
                        meta_rows=drow[mine], meta_tok=torch.arange(T).repeat_interleave(K).view(T, K)[mine],
                        meta_w=weights[mine]))
    return out
