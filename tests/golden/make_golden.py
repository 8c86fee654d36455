"""Generates tests/golden/*.json from the big-integer oracle (oracle/pyoracle.py).

The reference cannot be built or imported in this environment (Rust crate, no toolchain), so
these vectors are outputs of the restatement, pinned so that later changes to either oracle or
to the CUDA path are caught.  Run:  python tests/golden/make_golden.py
"""
import json
import os
import random
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import pyoracle as o  # noqa: E402


def hx(v):
    return "%064x" % v


def sumcheck_case(label, tables):
    n = len(tables[0]).bit_length() - 1
    t = o.Transcript(label)
    p = o.LinearSumcheckProver(n, len(tables), t)
    pr = p.prove(tables, t)
    return {"label": label.decode(), "tables": [[hx(v) for v in tb] for tb in tables],
            "round_messages": [[hx(v) for v in m] for m in pr.round_messages],
            "challenges": [hx(v) for v in p.challenges], "final_eval": hx(pr.final_eval),
            "tail": hx(t.challenge_scalar(b"after"))}


def main():
    rnd = random.Random(20240)
    out = {"merlin": {}, "linear": [], "sparse_dense": [], "sparse_bool": [], "poly": {}}
    t = o.Transcript.__new__(o.Transcript)
    t.strobe = o.Strobe128(b"Merlin v1.0")
    t.append_message(b"dom-sep", b"test protocol")
    t.append_message(b"some label", b"some data")
    out["merlin"]["simple"] = t.challenge_bytes(b"challenge", 32).hex()
    # hand-checkable tables of tests/test_linear_sumcheck.rs, then random ones
    out["linear"].append(sumcheck_case(b"sumcheck", [[1, 1, 1, 1], [1, 1, 1, 1]]))
    out["linear"].append(sumcheck_case(b"sumcheck", [[0, 1, 0, 1], [0, 0, 1, 1]]))
    out["linear"].append(sumcheck_case(b"sumcheck", [[0, 1]]))
    for n, ell in [(3, 2), (4, 3), (5, 4), (6, 1), (8, 2)]:
        out["linear"].append(sumcheck_case(b"sumcheck", [[rnd.randrange(o.R_MOD) for _ in range(1 << n)] for _ in range(ell)]))
    for n, nnz in [(4, 3), (7, 20), (9, 64)]:
        idx = sorted(rnd.sample(range(1 << n), nnz))
        vals = [o.fr_from_int(rnd.randrange(-128, 128)) for _ in idx]
        dense = [rnd.randrange(o.R_MOD) for _ in range(1 << n)]
        t = o.Transcript(b"sd_sumcheck")
        p, pr = o.sparse_dense_prove(n, idx, vals, dense, t)
        out["sparse_dense"].append({"n": n, "idx": idx, "vals": [hx(v) for v in vals], "dense": [hx(v) for v in dense],
                                    "round_messages": [[hx(v) for v in m] for m in pr.round_messages],
                                    "final_eval": hx(pr.final_eval), "tail": hx(t.challenge_scalar(b"after"))})
    for n, terms, k in [(5, 2, 6), (7, 3, 20)]:
        w = [rnd.randrange(o.R_MOD) for _ in range(terms)]
        pos = [rnd.sample(range(1 << n), k) for _ in range(terms)]
        pt = [rnd.randrange(o.R_MOD) for _ in range(n)]
        t = o.Transcript(b"range")
        sp = o.SparseBoolSumcheckProver(n, t)
        pr = sp.prove(w, pos, pt, t)
        out["sparse_bool"].append({"n": n, "weights": [hx(v) for v in w], "positions": pos, "eq_point": [hx(v) for v in pt],
                                   "round_messages": [[hx(v) for v in m] for m in pr.round_messages],
                                   "final_eval": hx(pr.final_eval), "tail": hx(t.challenge_scalar(b"after"))})
    f = [rnd.randrange(o.R_MOD) for _ in range(64)]
    pt = [rnd.randrange(o.R_MOD) for _ in range(6)]
    out["poly"] = {"f": [hx(v) for v in f], "point": [hx(v) for v in pt],
                   "eq": [hx(v) for v in o.evaluate_lagrange_basis(pt[:4])],
                   "fix_lsb_3": [hx(v) for v in o.fix_variables(f, pt[:3])],
                   "fix_right_2": [hx(v) for v in o.fix_variables_from_right(f, pt[:2])],
                   "mle": hx(o.evaluate_multilinear_extension(f, pt)),
                   "uniform_seed7": [hx(v) for v in o.gen_uniform_fr(7, 3, 5, 4)],
                   "small_seed7_bits8": [hx(v) for v in o.gen_small_fr(7, 3, 5, 8, 8)]}
    with open(os.path.join(HERE, "sumcheck.json"), "w") as fh:
        json.dump(out, fh, indent=0)
    print("wrote", os.path.join(HERE, "sumcheck.json"))


if __name__ == "__main__":
    main()
