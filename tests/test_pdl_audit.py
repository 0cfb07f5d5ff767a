"""Source audit: a kernel launched with programmatic stream serialization may start before its predecessor has
finished, so every such kernel has to execute griddepcontrol.wait (pdl_wait) before touching dependent memory.
Kernels whose launch carries the attribute are those launched through launch_pdl / launch_pdl_cluster and the FP4
GEMM (explicit attribute)."""
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _kernel_body(src: str, name: str) -> str:
    m = re.search(r"__global__[^{;]*\b" + re.escape(name) + r"\s*\([^{]*\{", src, re.S)
    assert m, name
    body = src[m.end():]
    nxt = body.find("__global__")
    return body if nxt < 0 else body[:nxt]


def test_every_pdl_launched_kernel_waits_for_its_predecessor():
    seen = 0
    for path in sorted(glob.glob(os.path.join(ROOT, "csrc", "*.cu"))):
        src = open(path).read()
        names = set(re.findall(r"launch_pdl(?:_cluster)?\(\s*([A-Za-z_0-9]+)", src))
        if "cudaLaunchAttributeProgrammaticStreamSerialization" in src:
            names |= set(re.findall(r"cudaLaunchKernelEx\(&cfg,\s*([A-Za-z_0-9]+)", src))
        for n in names:
            if n == "kern":          # gemm_tc: launched as an ordinary dependent (no attribute), still waits
                continue
            body = _kernel_body(src, n)
            assert "pdl_wait()" in body, (os.path.basename(path), n)
            seen += 1
    assert seen >= 15
