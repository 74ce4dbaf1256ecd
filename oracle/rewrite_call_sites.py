"""TEST INFRASTRUCTURE. Rewrites the 15 linear-layer launch sites of the reference's src/train.cu
(forward :356,360,365,369,376; backward :404,405,424,425,429,430,436,437,441,442) into calls of the
host launchers that include/compat/gpt2/layers/mlp.h provides under the same names:

    mlp_forward<TILE_SIZE><<<MLP_FORWARD_GRID(N, B, S), MLP_BLOCK_DIM, MLP_SHARED_MEM_SIZE>>>(args)
 -> mlp_forward<TILE_SIZE>(args)

Nothing else in the file changes. The output is written where oracle/Makefile asks (under oracle/_ref/,
which is not committed); the reference's source is read from where its tree is mounted.

    python oracle/rewrite_call_sites.py <reference>/src/train.cu <output.cu>
"""
import re
import sys

SITE = re.compile(r"(mlp_(?:forward|backward_input|backward_weight)<TILE_SIZE>)\s*<<<.*?>>>\s*\(", re.S)
EXPECTED = {"mlp_forward<TILE_SIZE>": 5, "mlp_backward_input<TILE_SIZE>": 5, "mlp_backward_weight<TILE_SIZE>": 5}


def rewrite(text):
    counts = {}

    def one(m):
        counts[m.group(1)] = counts.get(m.group(1), 0) + 1
        return m.group(1) + "("

    out = SITE.sub(one, text)
    if counts != EXPECTED:
        raise SystemExit(f"expected {EXPECTED} launch sites, found {counts}")
    return out


if __name__ == "__main__":
    if len(sys.argv) != 3:
        raise SystemExit(__doc__)
    with open(sys.argv[1]) as f:
        src = f.read()
    with open(sys.argv[2], "w") as f:
        f.write(rewrite(src))
