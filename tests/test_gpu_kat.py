"""The reference's own integration tests, run on the B200 backend through the C-ABI."""
import numpy as np
import pytest

import ref_programs
from helpers import b200, oracle, assert_ulp
from test_oracle_golden import check_against_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", sorted(ref_programs.ALL))
def test_reference_known_answers_on_b200(name):
    out = ref_programs.ALL[name](b200())
    check_against_golden(name, out)


@pytest.mark.parametrize("name", sorted(ref_programs.ALL))
def test_b200_matches_oracle_on_reference_programs(name):
    want = ref_programs.ALL[name](oracle())
    got = ref_programs.ALL[name](b200())
    for k in want:
        # these programs are a few ops deep; exp2/sin may differ by 2 ulp each and the chains amplify a little
        assert_ulp(f"{name}.{k}", got[k], want[k], 64)


def test_get_tensor_of_unkept_id_is_none():
    ad = ref_programs.ad
    ad.set_device(b200())
    ad.eager_dep_opt()
    x = ad.tensor([1.0, 2.0], [2])
    y = x * 2.0
    y.forward()
    y.val().keep()
    ad.execute()
    assert x.val().get().is_none                       # ValueData::none(), src/devices/opencl/device.rs:97-101
    np.testing.assert_array_equal(y.val().get().data, [2.0, 4.0])
