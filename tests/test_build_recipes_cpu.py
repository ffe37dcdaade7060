"""The xmake file is not run anywhere (xmake is not installed where this library is built), so the least that
is checked is that it lists exactly the sources the nvcc recipe compiles, and asks for sm_100a only."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_xmake_lists_the_sources_the_nvcc_recipe_compiles():
    from infinicore_b200 import build

    text = (ROOT / "xmake.lua").read_text()
    listed = set(re.findall(r'csrc \.\. "/([\w/]+\.cu)"', text))
    assert listed == set(build.RT_SOURCES) | set(build.OP_SOURCES) | set(build.CCL_SOURCES)
    for src in listed:
        assert (build.CSRC / src).is_file(), src
    assert 'add_cugencodes("arch=compute_100a,code=sm_100a")' in text
    assert not re.search(r"sm_[5-9]\d", text), "one architecture only"
    assert build.ARCH_FLAGS == ["-gencode", "arch=compute_100a,code=sm_100a"]
