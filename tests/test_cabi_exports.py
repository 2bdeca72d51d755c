"""The native library loads without a GPU and exports every entry point that include/*.h declares."""
import re
import subprocess

import pytest

from shield_sisa_b200 import binding
from tests.helpers import ROOT

DECL = re.compile(r"\b(shv_cuda_\w+|shv_box_\w+|shvb_\w+|shvk_\w+)\s*\(")


def declared_functions():
    names = set()
    for header in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
        for m in DECL.finditer(text):
            names.add(m.group(1))
    names -= {"shv_cuda_callback", "shv_box_ops"}       # typedefs, not exports
    return sorted(names)


@pytest.fixture(scope="module")
def built():
    from shield_sisa_b200 import build
    return build.build()


@pytest.mark.parametrize("experimental", [False, True])
def test_library_exports_every_declared_symbol(built, experimental):
    path = binding.library_path(experimental)
    out = subprocess.run(["nm", "-D", "--defined-only", str(path)], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    declared = declared_functions()
    assert len(declared) >= 40
    missing = [n for n in declared if n not in exported]
    assert not missing, f"declared in include/*.h but not exported: {missing}"
    # nothing but the public prefixes leaks out of the library
    stray = [n for n in exported if not n.startswith(("shv_cuda_", "shv_box_", "shvb_", "shvk_"))]
    assert not stray, stray


def test_library_loads_and_reports_revision(built):
    L = binding.load_library(True)
    rev = L.shv_cuda_compute_revision().decode()
    assert re.fullmatch(r"[0-9a-f]{16}", rev)
    opt = binding.Options()
    L.shv_cuda_default_options(opt)
    assert (opt.max_frames, opt.max_windows, opt.max_host_tokens, opt.token_slots, opt.use_graphs, opt.max_delay_us) == \
        (640, 512, 2048, 0, 1, 0)
