"""zkes_b200: B200-native proving hot path for zktransformer (BN254 sumcheck provers, multilinear
folds, KZH2/KZH3 commit/open MSMs) behind a C ABI.  This package is the thin host-side mirror
of the reference's Rust interface for that path; all arithmetic runs in libzkb200.so.

Names are resolved lazily so that `python -m zkes_b200.build` can run before the library exists."""
import importlib

_API = ("Context", "DenseMLPoly", "LinearSumcheckProver", "SumcheckProof", "Transcript",
        "SparseDenseSumcheckProver", "evaluate_lagrange_basis", "fix_variables_from_right", "permute_evals_by_ranges", "fix_variables_zkgpt",
        "SparseBoolSumcheckProver", "GeneralLinearSumcheckProver", "range_aux_accumulate", "range_table",
        "SumcheckVerifier")


def __getattr__(name):
    if name in _API:
        return getattr(importlib.import_module(".api", __name__), name)
    raise AttributeError(name)
