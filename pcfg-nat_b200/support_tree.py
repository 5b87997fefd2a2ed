"""Support-tree ("lemon tree") masks of PCFG-NAT, built without recursion.

Host-side mirror of ``BinaryTreeNode.get_mask(dim, left_tree_layer, src_upsample_scale)``
(fs_plugins/models/lemon_tree.py:92-119): the tree is a right-leaning main chain whose
nodes (except the first) each carry a complete binary left subtree of ``left_tree_layer``
levels; nodes are numbered in-order.  Node 0 is the left child of the first main-chain
node and doubles as the "no left child" slot.

Returned masks use the reference's convention: 1 (True) = NOT allowed.
"""
import torch


def max_left_of(left_tree_layer: int) -> int:
    """Number of nodes in one local left subtree (links.size(2) - 1 in the kernels)."""
    return 2 ** left_tree_layer - 1


def get_mask(dim: int, left_tree_layer: int, src_upsample_scale=None):
    """Returns (left_tree_mask [dim,dim], right_tree_mask [dim,dim], main_chain [dim]) as float tensors.

    ``left_tree_mask[a, j] == 0`` iff j lies in a's left subtree (or j == 0 and a >= 1);
    ``right_tree_mask[a, c] == 0`` iff c lies in a's right subtree; ``main_chain[a] == 1``
    for main-chain nodes.  ``src_upsample_scale`` is accepted for signature parity and is
    unused, exactly as in the reference (lemon_tree.py:41-59).
    """
    ml = max_left_of(left_tree_layer)
    step = ml + 1
    n_extra = (dim - 2) // step if dim >= 2 else 0  # main-chain nodes after the first
    total = 2 + n_extra * step if dim >= 2 else 0  # nodes that exist in the tree
    left = torch.ones(dim, dim)
    right = torch.ones(dim, dim)
    main = torch.zeros(dim)
    if dim >= 2:
        # first main-chain node: in-order position 1, left child = node 0
        for k in range(n_extra + 1):
            a = 1 + k * step
            main[a] = 1
            if k == 0:
                left[a, 0] = 0
            else:
                left[a, a - ml:a] = 0
            right[a, a + 1:total] = 0
        # complete binary subtrees in positions [a-ml, a-1]; iterate over (lo, hi) ranges
        for k in range(1, n_extra + 1):
            a = 1 + k * step
            stack = [(a - ml, a - 1)]
            while stack:
                lo, hi = stack.pop()
                if lo > hi:
                    continue
                mid = (lo + hi) // 2
                if lo <= mid - 1:
                    left[mid, lo:mid] = 0
                    stack.append((lo, mid - 1))
                if mid + 1 <= hi:
                    right[mid, mid + 1:hi + 1] = 0
                    stack.append((mid + 1, hi))
        left[1:, 0] = 0
    return left, right, main


def graph_length(src_length: int, src_upsample_scale: float, left_tree_layer: int) -> int:
    """Graph size the model allocates for a source of ``src_length`` tokens
    (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:319-323)."""
    return max(int(src_length * src_upsample_scale * (2 ** left_tree_layer)), 2) + 2
