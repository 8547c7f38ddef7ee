"""The CUDA engine against the reference's own known-answer vectors (and the oracle)."""
import pytest

from cudf_b200.types import TypeId
from oracle import oracle
from tests import helpers as H

CASES = [inst for case in H.load_golden() for inst in H.golden_instances(case)]


@pytest.mark.gpu
@pytest.mark.parametrize("inst", CASES, ids=[c[0] for c in CASES])
def test_engine_matches_reference_known_answers(inst):
    _, keys, vals, kind, ddof, policy, ekeys, evals = inst
    req = [(vals, [(kind, ddof)])]
    gkeys, gres = H.gpu_groupby([keys], req, policy)
    og, oe = H.sort_order(gkeys), H.sort_order([ekeys])
    H.assert_keys_equal(gkeys, [ekeys], og, oe)
    H.assert_column_equal(gres[0][0], evals, og, oe, 1e-15 if evals.type_id == TypeId.FLOAT64 else 1e-6, "values")
    H.assert_same_result((gkeys, gres), oracle.groupby([keys], req, policy), req)
