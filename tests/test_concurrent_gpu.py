"""Calls from several host threads on one context at once, as the reference opens its commitments from many rayon
workers (src/dag/mod.rs:893-936): KZH3 openings and fix_variables_from_right run concurrently on lanes of the
context and must return exactly what the same calls return one after another."""
import random
import threading

import pytest

import pyoracle as o
from zkes_b200 import DenseMLPoly, fix_variables_from_right, kzh
from zkes_b200._lib import ZK_OPT_LANES

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lanes", [4, 1])
def test_open_and_fold_from_four_threads(ctx, lanes):
    ctx.set_option(ZK_OPT_LANES, lanes)
    try:
        rnd = random.Random(99)
        n = 10
        xl, yl, zl = o.kzh3_degrees(n)
        tx = [rnd.randrange(1, o.R_MOD) for _ in range(1 << xl)]
        ty = [rnd.randrange(1, o.R_MOD) for _ in range(1 << yl)]
        tz = [rnd.randrange(1, o.R_MOD) for _ in range(1 << zl)]
        srs = kzh.KZHSRS.setup(ctx, 3, n, o.g1_mul(o.G1_GEN, 77), tx, ty, tau_z=tz)
        polys = [DenseMLPoly.from_evaluations([rnd.randrange(o.R_MOD) if i % 3 else o.fr_from_int(rnd.randrange(-99, 99))
                                               for i in range(1 << n)]) for _ in range(4)]
        coms = [kzh.commit(ctx, srs, p) for p in polys]
        points = [[rnd.randrange(o.R_MOD) for _ in range(n)] for _ in range(4)]
        tables = [DenseMLPoly.from_evaluations([rnd.randrange(o.R_MOD) for _ in range(1 << 15)]) for _ in range(4)]
        fixed = [[rnd.randrange(o.R_MOD) for _ in range(6)] for _ in range(4)]

        def work(i):
            _, d_y, c_y, f_star = kzh.kzh3_open(ctx, srs, points[i], coms[i], polys[i])
            folded = fix_variables_from_right(ctx, tables[i], fixed[i]).evaluations
            return d_y, c_y, f_star, folded

        serial = [work(i) for i in range(4)]
        # one of them against the oracle, so that "equal to the serial run" means "right"
        osrs = o.KZH3SRS(n, 77, tx, ty, tz)
        _, odx = o.kzh3_commit(osrs, polys[0].evaluations)
        _, ody, ocy, ofs = o.kzh3_open(osrs, points[0], odx, polys[0].evaluations)
        assert serial[0][:3] == (ody, ocy, ofs)
        assert serial[1][3] == o.fix_variables_from_right(tables[1].evaluations, fixed[1])

        results = [[None] * 4 for _ in range(4)]
        errors = []
        start = threading.Barrier(4)

        def runner(i):
            try:
                start.wait()
                for rep in range(4):
                    results[i][rep] = work(i)
            except Exception as e:  # noqa: BLE001
                errors.append(e)

        threads = [threading.Thread(target=runner, args=(i,)) for i in range(4)]
        before = ctx.launch_count
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        assert not errors, errors
        assert ctx.launch_count > before
        for i in range(4):
            for rep in range(4):
                assert results[i][rep] == serial[i], (i, rep)
        srs.close()
    finally:
        ctx.set_option(ZK_OPT_LANES, 4)
