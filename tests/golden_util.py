"""Helpers shared by the tests that read the committed golden fixtures."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, 'golden'))
import make_golden  # noqa: E402  (the generator also defines how inputs are regenerated from a seed)

CASES = make_golden.CASES
SEG_CASES = make_golden.SEG_CASES
TOK_CASES = make_golden.TOK_CASES
TOKDEC_CASES = make_golden.TOKDEC_CASES
ROLE_CASES = make_golden.ROLE_CASES
segment_roles = make_golden.segment_roles
ROW_STRIDE = make_golden.ROW_STRIDE


def load(name):
    """(case dict, fixture dict, (q, k, v, steps)) with the regenerated inputs checked against the stored checksums."""
    for table in (CASES, SEG_CASES, TOK_CASES, TOKDEC_CASES):
        if name in table:
            case = table[name]
    fx = dict(np.load(os.path.join(HERE, 'golden', name + '.npz')))
    q, k, v, steps = make_golden.golden_inputs(case)
    np.testing.assert_allclose(make_golden.checksum(q, k, v), fx['in_checksum'], rtol=0, atol=1e-6,
                               err_msg='seeded inputs no longer match the ones the fixture was made from')
    return case, fx, (q, k, v, steps)


def load_roles(name):
    """(case dict, fixture dict, hidden states of every call) of a role-sampling fixture."""
    case = ROLE_CASES[name]
    fx = dict(np.load(os.path.join(HERE, 'golden', name + '.npz')))
    xs = make_golden.role_inputs(case)
    np.testing.assert_allclose(make_golden.checksum(*xs), fx['in_checksum'], rtol=0, atol=1e-6,
                               err_msg='seeded inputs no longer match the ones the fixture was made from')
    return case, fx, xs
