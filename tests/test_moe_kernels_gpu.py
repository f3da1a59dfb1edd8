"""The mixture-of-experts FFN at the benchmark shape (512 routed experts, top-10 + shared, hidden 2048, expert FFN 512)
for the 24 rows of a configuration-5 verify pass, through the kernel-level C-ABI entry hp_moe_layer: bit for bit against
the CPU restatement (router GEMV, routing, per-(row, slot) expert GEMVs, SiLU, quantiser, slot-order combine) and,
for the routing, against the double-precision transcription of fn.hip:167-205."""
import numpy as np
import pytest
import torch

from hipster_b200 import kernels as K_, synth
from oracle import orc

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("n_expert,k,E,F,T", [(512, 10, 2048, 512, 24), (64, 4, 512, 256, 5), (512, 10, 2048, 512, 1)])
def test_moe_layer_bit_exact_vs_oracle(n_expert, k, E, F, T):
    rng = np.random.default_rng(n_expert + T)
    xn = rng.normal(0, 1, size=(T, E)).astype(np.float32)
    router = (rng.normal(0, 1, size=(n_expert + 1, E)) / np.sqrt(E)).astype(np.float32)     # router logits ~ N(0, 1)
    egu = synth.q4k_matrix(n_expert * 2 * F, E, seed=1).reshape(-1); edn = synth.q4k_matrix(n_expert * E, F, seed=2).reshape(-1)
    sgu = synth.q4k_matrix(2 * F, E, seed=3).reshape(-1); sdn = synth.q4k_matrix(E, F, seed=4).reshape(-1)
    d = lambda a: torch.from_numpy(a).cuda()
    ids, w, y = K_.moe_layer(d(xn), d(router), d(egu), d(edn), d(sgu), d(sdn), F, n_expert, k)
    K_.device_status()
    ids_o, w_o, y_o, lg = orc.moe_layer(xn, router, egu, edn, sgu, sdn, E, F, n_expert, k)
    assert np.array_equal(ids.cpu().numpy(), ids_o)
    assert np.array_equal(bits(w.cpu().numpy()), bits(w_o))
    assert np.array_equal(bits(y.cpu().numpy()), bits(y_o))
    # independent witness for the routing: same experts in the same order, weights within 1e-5 relative
    ids64, w64 = orc.ref64_moe_route(lg, n_expert, k)
    assert np.array_equal(ids64, ids_o)
    assert np.allclose(w_o, w64, rtol=1e-5, atol=0)


def test_router_ties_go_to_the_lower_expert_id():
    """Two experts with identical router rows get identical probabilities: the lower id must be ranked first."""
    n_expert, k, E, F, T = 64, 4, 512, 256, 3
    rng = np.random.default_rng(5)
    xn = rng.normal(0, 1, size=(T, E)).astype(np.float32)
    router = (rng.normal(0, 1, size=(n_expert + 1, E)) / np.sqrt(E)).astype(np.float32)
    router[40] = router[7] = 0.5 * xn[0] / np.linalg.norm(xn[0])          # both win row 0 with exactly equal logits
    egu = synth.q4k_matrix(n_expert * 2 * F, E, seed=1).reshape(-1); edn = synth.q4k_matrix(n_expert * E, F, seed=2).reshape(-1)
    sgu = synth.q4k_matrix(2 * F, E, seed=3).reshape(-1); sdn = synth.q4k_matrix(E, F, seed=4).reshape(-1)
    d = lambda a: torch.from_numpy(a).cuda()
    ids, w, y = K_.moe_layer(d(xn), d(router), d(egu), d(edn), d(sgu), d(sdn), F, n_expert, k)
    ids_o, w_o, y_o, _ = orc.moe_layer(xn, router, egu, edn, sgu, sdn, E, F, n_expert, k)
    assert list(ids_o[0][:2]) == [7, 40]
    assert np.array_equal(ids.cpu().numpy(), ids_o) and np.array_equal(bits(y.cpu().numpy()), bits(y_o))


def test_unit_form_of_the_expert_gemv_matches_too():
    """The one-warp-per-unit form of the expert GEMVs (taken when the quads' activation buffers do not fit in shared
    memory, or with HIPSTER_B200_MOE_UNITS set) must give the same bits: the switch is read once per process, so the
    parity test of the small shape runs again in a child process with it set."""
    import os, subprocess, sys
    if os.environ.get("HIPSTER_B200_MOE_UNITS"):
        pytest.skip("already inside the child process")
    env = dict(os.environ, HIPSTER_B200_MOE_UNITS="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_moe_kernels_gpu.py"), "-q", "-m", "gpu", "-k", "bit_exact and 64-4"],
                       env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "1 passed" in r.stdout
