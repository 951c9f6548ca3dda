"""Drop-in proof: the REFERENCE's own runtime (arena, tensor, node, op table, graph, scheduler,
compiled from its sources by oracle/Makefile into oracle/_ref/dropin_check) drives
libplast_b200.so for device = CUDA and its own CPU kernels for device = CPU on the same graphs;
the binary compares the two (oracle/dropin_check.c) and exits 0 when they agree."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

BIN = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "dropin_check"


@pytest.mark.skipif(not BIN.exists(), reason="oracle/_ref/dropin_check not built (reference sources absent at build time)")
def test_reference_runtime_drives_the_library():
    p = subprocess.run([str(BIN)], capture_output=True, text=True, timeout=120)
    print(p.stdout, p.stderr)
    assert p.returncode == 0, p.stdout + p.stderr
    assert "DROPIN OK" in p.stdout
    # A + b, relu(A + b), max(X.T); fused relu(A + b), row sums and chain against the node-by-node runs
    # ... and the gradients of the fused training chain against its nine backward nodes
    # ... and the row sums of the DAG replayed as one CUDA graph
    assert p.stdout.count("bit-exact") == 13          # + the four comparisons of the arena-fill runs
