"""TEST INFRASTRUCTURE ONLY.  Cuts the statement blocks that define the attention arithmetic out of
the Granite checkout's src/llm/transformer.mm into generated include files under oracle/_ref/
(git-ignored), so that oracle/ref_loops.cpp can compile the reference's OWN statements - not a
restatement - into oracle/_ref/libgranite_ref.so.  Nothing of the reference is copied into the
repository: the files this script writes are build products.

The blocks cannot be called where they stand: TransformerModel::attention() projects Q/K/V from
model weights and needs a model file, and transformer.mm does not compile without Metal.  Each
block, however, is self-contained over local variables (q_data, k_all, v_all, scale, total_seq,
context, ...), so a wrapper function whose parameters carry those names can include it verbatim.

Blocks are found by anchor comments (unique in the file) and cross-checked against the line
numbers they had when the citations in this repository were written; a checkout where an anchor
moved by more than a few lines, or is missing or ambiguous, fails the build loudly instead of
slicing something else.

Usage: python slice_reference.py <granite checkout> <output directory>
"""
from __future__ import annotations

import sys
from pathlib import Path

SOURCE = "src/llm/transformer.mm"

# name -> (first-line anchor, last-line anchor, include the last line?, expected first line, expected last line)
BLOCKS = {
    # TransformerModel::attention: GQA mapping, causal scores, three-pass softmax, P.V (`context`)
    "attention_loop": ("    // Compute attention for each head (parallelized)", "    });  // End parallel_for", True, 1779, 1840),
    # TransformerModel::attention: whole-cache fp16 -> fp32 widening into [total_seq, Hkv, D]
    "attention_cache_widen": ("            // [1, num_kv_heads, total_seq, head_dim] -> [total_seq, num_kv_heads, head_dim]",
                              "            backend_->unmap_buffer(cached_k.buffer());", False, 1753, 1765),
    # TransformerModel::attention_tree: prefix + masked tree scores, softmax, P.V
    "tree_loop": ("    // Compute attention for each head", "    });  // End parallel_for", True, 2044, 2126),
    # TransformerModel::forward_tree: ancestor mask from the parent array
    "tree_mask": ("    // Build tree_mask only if using CPU path", "    // Create tensor from tokens [1, num_nodes]", False, 822, 841),
}
SLACK = 40  # lines an anchor may have moved before the slice is refused


def cut(lines: list[str], name: str) -> str:
    first_anchor, last_anchor, inclusive, want_first, want_last = BLOCKS[name]
    starts = [i for i, l in enumerate(lines) if l.rstrip("\n") == first_anchor]
    if len(starts) != 1:
        raise SystemExit(f"slice_reference: {name}: first-line anchor found {len(starts)} times, expected once")
    first = starts[0]
    last = next((i for i in range(first + 1, len(lines)) if lines[i].rstrip("\n") == last_anchor), None)
    if last is None:
        raise SystemExit(f"slice_reference: {name}: last-line anchor not found after line {first + 1}")
    if not inclusive:
        last -= 1
    if abs(first + 1 - want_first) > SLACK or abs(last + 1 - want_last) > SLACK:
        raise SystemExit(f"slice_reference: {name}: found at {first + 1}-{last + 1}, expected about {want_first}-{want_last}")
    return "".join(lines[first:last + 1])


def main(ref_dir: str, out_dir: str) -> None:
    src = Path(ref_dir) / SOURCE
    lines = src.read_text().splitlines(keepends=True)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    for name in BLOCKS:
        body = cut(lines, name)
        header = f"// GENERATED from {SOURCE} of the Granite checkout by oracle/slice_reference.py - a build product, never committed.\n"
        (out / f"{name}.inc").write_text(header + body)


if __name__ == "__main__":
    if len(sys.argv) != 3:
        raise SystemExit(__doc__)
    main(sys.argv[1], sys.argv[2])
