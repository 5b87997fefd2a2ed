"""Independent pure-Python / float64 restatements used to cross-check the C oracle.

``loss_two_term`` is the left-tree-layer-1 specialisation of the inside recurrence
(pcfg_loss.cu:149-213 with max_left == 1: of the four (j, b) combinations only
"no left child, j=0" and "leaf left child, j=1" are ever finite), written with torch in
float64 so autograd gives an independent gradient.  ``loss_bruteforce`` enumerates every
derivation explicitly.
"""
import itertools
import math

import torch

NEG = float("-inf")


def _lse(xs):
    """-inf-safe logsumexp of a list of 0-d tensors (torch.logsumexp gives NaN grads on all -inf)."""
    fin = [x for x in xs if x.item() != NEG]
    if not fin:
        return torch.tensor(NEG, dtype=torch.float64)
    return torch.logsumexp(torch.stack(fin), 0)


def loss_two_term(match, links, m, n):
    """S[0][0] for one sentence; match [L,T], links [L,2,L] float64 tensors (may require grad)."""
    M = m // 2  # main-chain nodes a = 2*ai+1 < m
    last = (m - 2) // 2
    S = [[torch.tensor(NEG, dtype=torch.float64) for _ in range(n + 2)] for _ in range(M)]
    S[last][n - 1] = match[m - 1, n - 1]
    for t in range(n - 2, -1, -1):
        for ai in range(M):
            a = 2 * ai + 1
            terms = []
            for ci in range(ai + 1, M):
                c = 2 * ci + 1
                terms.append(links[a, 0, c] + S[ci][t + 1] + match[a, t])
                if a >= 3 and t + 1 < n:
                    terms.append(links[a, 1, c] + S[ci][t + 2] + match[a - 1, t] + match[a, t + 1])
            S[ai][t] = _lse(terms)
    return S[0][0]


def loss_bruteforce(match, links, m, n):
    """log of the sum over all derivations, enumerated one by one (tiny m only)."""
    M = m // 2
    mains = [2 * i + 1 for i in range(M)]
    if mains[-1] != m - 1:
        return NEG
    inner = mains[1:-1]
    total = []
    for r in range(len(inner) + 1):
        for sub in itertools.combinations(inner, r):
            chain = [1] + list(sub) + [m - 1]
            k = len(chain)
            # nodes chain[1..k-2] may take a leaf left child; node 1 and the last node cannot
            for uses in itertools.product([0, 1], repeat=max(k - 2, 0)):
                use = [0] + list(uses) + [0]
                if sum(use) + k != n:
                    continue
                lp, t = 0.0, 0
                for i, a in enumerate(chain):
                    if use[i]:
                        lp += float(match[a - 1, t])
                        t += 1
                    lp += float(match[a, t])
                    t += 1
                    if i + 1 < k:
                        lp += float(links[a, use[i], chain[i + 1]])
                if lp != NEG and not math.isnan(lp):
                    total.append(lp)
    if not total:
        return NEG
    mx = max(total)
    return mx + math.log(sum(math.exp(x - mx) for x in total))


def glance_select(path, pred_tokens, tgt_tokens, prev_output_tokens, target_length, noise, context_p,
                  strategy="number-random", uniform=None):
    """Torch restatement of the glancing sampler (fs_plugins/criterions/nat_pcfg_loss.py:216-267) with the random
    draws given: ``noise`` = the reference's torch.randn, ``uniform`` = its torch.rand ([B] for "cmlm", [B, L] for
    strategy None).  Pinned against the reference's own function by tests/golden/host_criterion.npz."""
    import torch

    B, L = path.shape
    T = tgt_tokens.shape[1]
    path = path.clone()
    aligned = path >= 0
    path[(path + 1 >= T + 1) | (path + 1 < 0)] = -1
    matchmask = torch.zeros(B, T + 1, L, dtype=torch.bool).scatter_(1, path.unsqueeze(1) + 1, True)[:, 1:]
    oracle = tgt_tokens.gather(-1, path.clip(min=0))
    same_num = ((pred_tokens == oracle) & aligned).sum(1)
    if strategy is None:
        keep_prob = ((target_length - same_num) / target_length * context_p).unsqueeze(-1) * aligned.float()
        keep = uniform < keep_prob
        glance_nums = keep.sum(1)
    else:
        prob = noise.clone().masked_fill_(~aligned, -100)
        if strategy == "cmlm":
            glance_nums = (target_length * uniform + 0.5).to(torch.long)
        else:
            glance_nums = ((target_length - same_num) * context_p + 0.5).to(torch.long)
        thresh = prob.sort(descending=True)[0].gather(-1, (glance_nums - 1).clip(min=0).unsqueeze(-1)).squeeze(-1)
        thresh = thresh.masked_fill(glance_nums == 0, 100)
        keep = prob >= thresh.unsqueeze(-1)
    glat_prev = prev_output_tokens.masked_fill(keep, 0) + oracle.masked_fill(~keep, 0)
    return {"matchmask": matchmask, "oracle": oracle, "same_num": same_num, "glance_num": glance_nums,
            "keep_word_mask": keep, "glat_prev_output_tokens": glat_prev}


def criterion_draws(strategy, seed, B, L):
    """The draws torch's seeded global generator gives the reference's glat_function, in its order
    (nat_pcfg_loss.py:233, :241-243, :248): (noise [B, L] or None, uniform or None)."""
    import torch

    torch.manual_seed(seed)
    if strategy is None:
        return None, torch.rand(B, L)
    noise = torch.randn(B, L, dtype=torch.float)
    uniform = torch.rand(B, dtype=torch.float) if strategy == "cmlm" else None
    return noise, uniform


def force_emit(match_eos_masked, matchmask, keep_word_mask):
    """(masked emissions, gradient mask) of the force-emit step (nat_pcfg_loss.py:116-121): a revealed node keeps
    only the entry of its aligned target position and passes no gradient."""
    import torch

    keep = keep_word_mask.unsqueeze(-1)
    mm = matchmask.transpose(1, 2)
    out = torch.where(keep & ~mm, torch.full_like(match_eos_masked, NEG), match_eos_masked)
    return out, (~keep).expand_as(match_eos_masked)


def extract_links(q, kl, kr, gate_logits, prev_output_tokens, pad, left_mask, right_mask, main_chain):
    """Torch restatement (max_left == 1) of what the model's extract_links computes
    (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:140-201), from the projected link features
    q, kl, kr [B, L, heads, D] and gate logits [B, L, heads]:
    links[b, a, k, c] = logsumexp_h( log_softmax_{(k, c)}( (ab + bc) + ac ) + log_softmax_h(gates) )."""
    import torch

    B, L, H, D = q.shape
    q, kl, kr = q.float(), kl.float(), kr.float()
    scale = D ** 0.5
    nonpad = prev_output_tokens.ne(pad)
    left_ok = nonpad[:, None, :] & ~left_mask.bool()[None, :L, :L]                      # [B, a, j]
    right_ok = nonpad[:, None, :] & ~right_mask.bool()[None, :L, :L] & main_chain.bool()[None, None, :L]
    use = left_ok.any(-1) & right_ok.any(-1)                                             # [B, a]
    left_idx = torch.stack([torch.zeros(L, dtype=torch.long), (torch.arange(L) - 1).clamp(min=0)], -1)  # [a, k]
    kl_opt = kl[:, left_idx]                                                             # [B, a, k, H, D]
    ab = torch.einsum("bahd,bakhd->bakh", q, kl_opt) / scale
    ab_ok = torch.gather(left_ok, 2, left_idx[None].expand(B, -1, -1))                   # [B, a, k]
    ab = ab.masked_fill(~ab_ok[..., None] & use[:, :, None, None], float("-inf"))
    bc = torch.einsum("bakhd,bchd->bakch", kl_opt, kr) / scale
    ac = torch.einsum("bahd,bchd->bach", q, kr) / scale
    ac = ac.masked_fill(~right_ok[..., None] & use[:, :, None, None], float("-inf"))
    abc = (ab[:, :, :, None, :] + bc) + ac[:, :, None, :, :]                             # [B, a, k, c, H]
    lp = torch.log_softmax(abc.reshape(B, L, 2 * L, H), 2)
    lg = torch.log_softmax(gate_logits.float(), -1)
    links = torch.logsumexp(lp + lg[:, :, None, :], -1).view(B, L, 2, L)
    return links.masked_fill(~use[:, :, None, None], float("-inf"))


def lookahead_decode(links, ob_lprob, tokens, output_length, left_tree_mask, pad, beta=1.0, lookahead=True):
    """Restatement of the model's "lookahead" / "greedy" decoding
    (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:419-482), every sentence with its own
    log-probabilities.  Returns the per-sentence token lists.  Pinned against the reference's own block by
    tests/golden/host_lookahead.npz."""
    import torch

    B, L = links.shape[0], links.shape[1]
    if lookahead:
        left = torch.stack([torch.zeros(L, dtype=torch.long), (torch.arange(L) - 1).clamp(min=0)], -1)  # [a, k]
        look = (links + ob_lprob[:, None, None, :] * beta) + (ob_lprob[:, left] * beta)[..., None]
    else:
        look = links
    idx = look.reshape(B, L, 2 * L).max(-1)[1].tolist()
    rows = []
    for i in range(B):
        length = int(output_length[i])
        now, stack, res = 1, [], []
        while (now < length and now != 0) or stack:
            while now < length and now != 0:
                stack.append(now)
                k = idx[i][now] // L
                lft = 0 if k == 0 else now - k
                if left_tree_mask[now][lft]:
                    break
                now = lft
            now = stack.pop()
            t = int(tokens[i][now])
            if t != pad:
                res.append(t)
            now = idx[i][now] % L
        rows.append(res)
    return rows
