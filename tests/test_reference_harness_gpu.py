"""The reference's own tests, unmodified, against this library: test/infiniop/paged_attention.py,
paged_caching.py, paged_attention_prefill.py, rope.py and kv_caching.py with the reference's ctypes harness
(staged under oracle/_ref/test_infiniop/ when the reference checkout was at hand), $INFINI_ROOT pointing at this
library's lib/ folder.  Each script builds its own inputs, calls the operator through the C ABI exactly as the
reference's CI does, checks the result against its torch implementation with its own tolerances and prints
"Test passed!"."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
HARNESS = ROOT / "oracle" / "_ref" / "test_infiniop"
SCRIPTS = ["paged_attention.py", "paged_caching.py", "paged_attention_prefill.py", "rope.py", "kv_caching.py"]


@pytest.mark.parametrize("script", SCRIPTS)
def test_reference_test_script_passes_on_this_library(script):
    if not (HARNESS / script).is_file():
        pytest.skip("the reference's test scripts are not staged (oracle/_ref/test_infiniop)")
    env = dict(os.environ)
    env["INFINI_ROOT"] = str(ROOT / "infinicore_b200")
    for k in [k for k in env if k.startswith("INFINIOP_")]:
        env.pop(k)
    res = subprocess.run([sys.executable, str(ROOT / "tests" / "ref_harness.py"), script, "--nvidia"], env=env, capture_output=True,
                         text=True, timeout=1200, cwd=str(HARNESS))
    tail = (res.stdout + res.stderr)[-3000:]
    assert res.returncode == 0, tail
    assert "Test passed!" in res.stdout, tail
