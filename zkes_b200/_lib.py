"""ctypes binding of libzkb200.so (see include/zkb200.h).  There is no CPU fallback: if the
library is missing or fails to load, importing this module raises."""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_int, c_size_t, c_uint8, c_uint32, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libzkb200.so")

ZK_MEM_HOST, ZK_MEM_DEVICE = 0, 1
ZK_OPT_DEVICE_TAIL = 1
ZK_OPT_REPLICATE_LOG = 2
ZK_OPT_PEER_EXCHANGE = 3
ZK_OPT_EXCHANGE_WAIT_MS = 4
ZK_OPT_LANES = 5
ZK_OPT_AHEAD_LOG = 6
ZK_OK, ZK_ERR_ARG, ZK_ERR_OOM, ZK_ERR_CUDA, ZK_ERR_TIMEOUT, ZK_ERR_FS_CALLBACK, ZK_ERR_COMM = 0, -1, -2, -3, -4, -5, -6

FS_ROUND_FN = ctypes.CFUNCTYPE(c_int, c_void_p, POINTER(c_uint64), c_uint32, POINTER(c_uint64))

_u64p = POINTER(c_uint64)
_u8p = POINTER(c_uint8)

# name -> (restype, argtypes); every symbol include/zkb200.h declares appears here.
SIGNATURES = {
    "zk_init": (c_int, [c_int, POINTER(c_void_p)]),
    "zk_free": (None, [c_void_p]),
    "zk_last_error": (c_char_p, []),
    "zk_launch_count": (c_uint64, [c_void_p]),
    "zk_set_option": (c_int, [c_void_p, c_int, c_int]),
    "zk_stream": (c_void_p, [c_void_p]),
    "zk_profile_enable": (c_int, [c_void_p, c_int]),
    "zk_profile_get": (c_int, [c_void_p, c_int, POINTER(c_uint64), POINTER(ctypes.c_double),
                               POINTER(ctypes.c_double)]),
    "zk_device_alloc": (c_int, [c_void_p, c_size_t, POINTER(c_void_p)]),
    "zk_device_free": (c_int, [c_void_p, c_void_p]),
    "zk_device_copy": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_size_t]),
    "zk_device_sync": (c_int, [c_void_p]),
    "zk_transcript_new": (c_void_p, [c_char_p, c_size_t]),
    "zk_transcript_clone": (c_void_p, [c_void_p]),
    "zk_transcript_free": (None, [c_void_p]),
    "zk_transcript_append_message": (None, [c_void_p, c_char_p, c_size_t, c_char_p, c_size_t]),
    "zk_transcript_append_u64": (None, [c_void_p, c_char_p, c_size_t, c_uint64]),
    "zk_transcript_append_scalar": (None, [c_void_p, c_char_p, c_size_t, c_void_p]),
    "zk_transcript_challenge_bytes": (None, [c_void_p, c_char_p, c_size_t, c_void_p, c_size_t]),
    "zk_transcript_challenge_scalar": (None, [c_void_p, c_char_p, c_size_t, c_void_p]),
    "zk_sumcheck_linear_prove": (c_int, [c_void_p, c_uint32, c_uint32, POINTER(c_void_p), c_int, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "zk_sumcheck_sparse_dense_prove": (c_int, [c_void_p, c_uint32, c_uint64, c_void_p, c_void_p, c_void_p, c_int,
                                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p]),
    "zk_sumcheck_verify": (c_int, [c_void_p, c_uint32, c_uint32, c_void_p, c_uint32, c_uint32, c_void_p, c_void_p,
                                   c_void_p, POINTER(c_int), POINTER(c_uint32)]),
    "zk_fix_from_right": (c_int, [c_void_p, c_uint32, c_void_p, c_int, c_uint32, c_void_p, c_void_p, c_int]),
    "zk_kzh_verify_g1": (c_int, [c_void_p, c_void_p, c_void_p, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p]),
    "zk_g1_compress": (c_int, [c_void_p, c_void_p, c_int, c_uint64, c_void_p, c_int]),
    "zk_g1_decompress": (c_int, [c_void_p, c_void_p, c_int, c_uint64, c_void_p, c_int]),
    "zk_kzh_open_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_uint32, c_void_p, c_void_p,
                                    c_void_p, c_void_p]),
    "zk_mle_eval": (c_int, [c_void_p, c_uint32, c_void_p, c_int, c_void_p, c_void_p]),
    "zk_range_aux_accumulate": (c_int, [c_void_p, c_uint32, c_void_p, c_uint64, c_void_p, c_void_p, c_int, c_void_p, c_uint32,
                                        c_void_p, c_int, c_void_p]),
    "zk_range_table": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_int]),
    "zk_permute_by_ranges": (c_int, [c_void_p, c_uint32, c_uint32, c_void_p, c_int, c_uint32, c_void_p, c_void_p, c_int]),
    "zk_fix_variables_int": (c_int, [c_void_p, c_uint32, c_void_p, c_int, c_uint32, c_void_p, c_void_p, c_int]),
    "zk_eq_table": (c_int, [c_void_p, c_uint32, c_void_p, c_void_p, c_int]),
    "zk_msm_g1": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int, c_uint64, c_void_p, c_int]),
    "zk_msm_g1_batched": (c_int, [c_void_p, c_void_p, c_int, c_uint64, c_void_p, c_int, c_uint64, c_void_p, c_int]),
    "zk_msm_g1_gather": (c_int, [c_void_p, c_void_p, c_int, c_uint64, c_void_p, c_void_p, c_int, c_uint64, c_void_p,
                                 c_int]),
    "zk_g1_normalize": (c_int, [c_void_p, c_void_p, c_int, c_uint64, c_void_p, c_int]),
    "zk_msm_last_stats": (c_int, [c_void_p, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_uint64),
                                  POINTER(c_uint64)]),
    "zk_msm_work": (c_int, [c_void_p, POINTER(c_uint64), POINTER(c_uint64), POINTER(c_uint64), c_int]),
    "zk_kzh_srs_setup": (c_int, [c_void_p, c_int, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 POINTER(c_void_p)]),
    "zk_kzh_srs_upload": (c_int, [c_void_p, c_int, c_uint32, c_void_p, c_void_p, c_void_p, c_int, POINTER(c_void_p)]),
    "zk_kzh_srs_free": (None, [c_void_p, c_void_p]),
    "zk_kzh_srs_shape": (c_int, [c_void_p, POINTER(c_uint32), POINTER(c_uint32), POINTER(c_uint32)]),
    "zk_kzh_srs_read": (c_int, [c_void_p, c_void_p, c_int, c_uint64, c_uint64, c_void_p]),
    "zk_kzh_commit": (c_int, [c_void_p, c_void_p, c_uint32, c_void_p, c_int, c_void_p, c_void_p]),
    "zk_kzh2_open": (c_int, [c_void_p, c_void_p, c_uint32, c_void_p, c_int, c_void_p, c_uint32, c_void_p]),
    "zk_kzh3_open": (c_int, [c_void_p, c_void_p, c_uint32, c_void_p, c_int, c_void_p, c_uint32, c_void_p, c_void_p,
                             c_void_p, c_void_p]),
    "zk_sparse_kzh_commit": (c_int, [c_void_p, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "zk_sparse_kzh2_open": (c_int, [c_void_p, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_uint32, c_void_p]),
    "zk_sparse_kzh3_open": (c_int, [c_void_p, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_uint32, c_void_p,
                                    c_void_p, c_void_p, c_void_p]),
    "zk_fold_lsb_static": (c_int, [c_uint32, c_void_p, c_uint32, c_void_p, c_void_p, c_void_p]),
    "zk_gen_gauss_fr": (c_int, [c_void_p, c_uint64, c_uint64, c_uint64, c_uint64, c_int, c_void_p]),
    "zk_weighted_fold_from_right": (c_int, [c_void_p, c_uint32, c_void_p, c_int, c_uint32, c_void_p, c_int, c_void_p,
                                            c_int]),
    "zk_gen_uniform_fr": (c_int, [c_void_p, c_uint64, c_uint64, c_uint64, c_uint64, c_void_p]),
    "zk_gen_small_fr": (c_int, [c_void_p, c_uint64, c_uint64, c_uint64, c_uint64, c_int, c_void_p]),
    "zk_sumcheck_sparse_bool_prove": (c_int, [c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "zk_sumcheck_sparse_bool_prove_sharded": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, c_void_p, c_void_p, c_void_p,
                                                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "zk_sumcheck_general_prove": (c_int, [c_void_p, c_uint32, c_uint32, c_uint32, c_void_p, POINTER(c_void_p), c_void_p,
                                          c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "zk_comm_unique_id": (c_int, [c_void_p]),
    "zk_comm_init": (c_int, [c_void_p, c_int, c_int, c_void_p, POINTER(c_void_p)]),
    "zk_comm_free": (None, [c_void_p, c_void_p]),
    "zk_comm_peer_exchange": (c_int, [c_void_p]),
    "zk_comm_wait_selftest": (c_int, [c_void_p, c_uint32]),
    "zk_round_times": (c_int, [c_void_p, c_void_p, c_uint32, c_void_p]),
    "zk_sumcheck_linear_prove_sharded": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, POINTER(c_void_p), c_int,
                                                 c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "zk_sumcheck_sparse_dense_prove_sharded": (c_int, [c_void_p, c_void_p, c_uint32, c_uint64, c_void_p, c_void_p,
                                                       c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                                       c_void_p, c_void_p, c_void_p]),
    "zk_msm_g1_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_uint64, c_void_p]),
    "zk_fix_from_right_sharded": (c_int, [c_void_p, c_void_p, c_uint32, c_void_p, c_int, c_uint32, c_void_p, c_void_p]),
    "zk_kzh_srs_setup_sharded": (c_int, [c_void_p, c_int, c_int, c_int, c_uint32, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, POINTER(c_void_p)]),
    "zk_kzh_commit_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "zk_microbench": (c_int, [c_void_p, c_int, c_int, c_int, c_int, POINTER(ctypes.c_float),
                              POINTER(ctypes.c_double)]),
    "zk_fold_lsb": (c_int, [c_void_p, c_uint32, c_void_p, c_int, c_uint32, c_void_p, c_void_p, c_int]),
}


def load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m zkes_b200.build` (there is no CPU fallback)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()


class ZkError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib.zk_last_error()
        super().__init__(f"{where}: status {code}: {msg.decode() if msg else ''}")


def check(code: int, where: str):
    if code != ZK_OK:
        raise ZkError(code, where)
