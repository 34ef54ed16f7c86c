"""Second checker: the reference's OWN CUDA path (Trainer / Mapper with UseGPU = true and the CudaLib kernels,
compiled unmodified for sm_100a into oracle/_ref/libpink_ref_cuda.so), run on the same GPU in a process of its own.

Its float arithmetic is not defined at source level (nvcc contracts its interpolation and update to FMA, the
distance is a 256-way tree sum of scaled partials), so agreement is asserted up to those effects: mapped distances
within a small relative tolerance, and wherever its best transform or best matching unit differs from this
library's, the two candidates must be near-ties in this library's own exact distance matrix.  Geometry of the
10 x 10 / 44 x 44 / 64 x 64-image configuration: the rotated window stays inside the image, so the reference's
interpolation never touches the row past the image."""
import numpy as np
import pytest

import oracle as O
from pink_b200 import capi, engine
from pink_b200.synthetic import blob_images, mt19937_uniform
from test_gpu_stages import _distance, _rotate

pytestmark = pytest.mark.gpu

S, IDIM, ND, ED, R = 10, 64, 44, 31, 360
# (distance tolerance, near-tie tolerance on the squared distance)
TOL = {2: (3e-3, 1e-2), 0: (1e-4, 2e-4)}


@pytest.mark.parametrize("mode", [2, 0])
def test_against_the_reference_cuda_path(cuda, mode):
    if not O.have_ref_cuda():
        pytest.skip("the reference's CUDA path was not built (its source tree was absent at build time)")
    N, T = S * S, 2 * R
    som = mt19937_uniform(N * ND * ND, 1234).reshape(N, ND, ND)
    imgs = blob_images(4, IDIM, 1, seed=1001).reshape(4, IDIM, IDIM)
    ref = O.ref_cuda_run("map", som, imgs, 0, S, S, IDIM, ND, ED, R, True, mode)
    with engine.Engine(N, 1, IDIM, ND, ED, R, True, mode) as eng:
        eng.set_som(som)
        dist, rot = eng.map(imgs)
    tol_d, tol_tie = TOL[mode]
    np.testing.assert_allclose(dist, ref["dist"], rtol=tol_d)
    # this library's full matrix for the near-tie rule
    a = O.crop_quantize(som.reshape(N, 1, ND, ND), ED, mode)
    _, b0, _, _, K, _ = _rotate(cuda, capi, imgs.reshape(4, 1, IDIM, IDIM), 1, IDIM, ND, ED, R, True, mode)
    disagree = 0
    for i in range(len(imgs)):
        b = b0[i * T:(i + 1) * T, :K]
        _, mat = _distance(cuda, capi, a, np.ascontiguousarray(b), mode)
        m = mat[0].astype(np.float64)
        ours, theirs = rot[i], ref["rot"][i]
        diff = np.flatnonzero(ours != theirs)
        disagree += len(diff)
        # where the transforms differ, the reference's choice is a near-tie of ours in our exact matrix
        assert (m[diff, theirs[diff]] <= m[diff, ours[diff]] * (1 + tol_tie)).all()
        # and so is its best matching unit
        bmu_o, bmu_r = int(np.argmin(dist[i])), int(np.argmin(ref["dist"][i]))
        assert bmu_o == bmu_r or dist[i][bmu_r] <= dist[i][bmu_o] * (1 + tol_d)
    assert disagree <= 0.05 * len(imgs) * N               # near-ties are the exception, not the rule

    # one training step from the same map: same unit, and the same new weights up to the FMA contraction of the
    # reference's kernels, for every neuron whose best transform agrees
    F = engine.update_factors(capi.LAYOUT_CARTESIAN, S, S, capi.FUNC_GAUSSIAN, 1.1, 0.2)
    trained = O.ref_cuda_run("train", som, imgs[:1], 0, S, S, IDIM, ND, ED, R, True, mode)["som"]
    with engine.Engine(N, 1, IDIM, ND, ED, R, True, mode) as eng:
        eng.set_som(som)
        eng.set_update_factors(F)
        eng.train(imgs[:1])
        bmu = int(eng.bmu_log(1)[0])
        got = eng.get_som(np.zeros_like(som.reshape(N, -1))).reshape(N, ND, ND)
    if bmu == int(np.argmin(ref["dist"][0])):
        same = rot[0] == ref["rot"][0]
        np.testing.assert_allclose(got[same], trained[same], rtol=2e-5, atol=2e-6)
