"""Metrics against closed forms / plain torch (model: the reference's ``test/metrics`` suite)."""
import math

import numpy as np
import pytest
import torch

from physicsnemo_b200.metrics.general import calibration, crps, ensemble_metrics as em, entropy, histogram as hist
from physicsnemo_b200.metrics.general import mse as mse_mod, power_spectrum as ps, reduction, relative_error as re
from physicsnemo_b200.metrics.general import wasserstein as ws
from physicsnemo_b200.metrics.climate import acc as acc_mod, efi as efi_mod, reduction as clim_red
from physicsnemo_b200.metrics.climate.loss import MSE_SSIM, SSIM
from physicsnemo_b200.metrics.climate.graphcast_loss import (CellAreaWeightedLossFunction,
                                                             CustomCellAreaWeightedLossFunction)
from physicsnemo_b200.metrics.cae import cfd, integral


def test_mse_rmse_relative():
    torch.manual_seed(0)
    p, t = torch.randn(4, 5, 6), torch.randn(4, 5, 6)
    assert torch.allclose(mse_mod.mse(p, t), ((p - t) ** 2).mean())
    assert torch.allclose(mse_mod.rmse(p, t, dim=1), ((p - t) ** 2).mean(1).sqrt())
    w = torch.rand(6)
    ref = ((p - t) ** 2 * w).sum(-1) / w.sum()
    assert torch.allclose(mse_mod.mse(p, t, dim=-1, weights=w), ref, atol=1e-6)
    r = re.relative_l2(p, t, reduction="none")
    assert torch.allclose(r, (p - t).flatten(1).norm(dim=1) / t.flatten(1).norm(dim=1), atol=1e-6)
    assert torch.allclose(re.relative_mse(p, t), (r ** 2).mean(), atol=1e-6)
    with pytest.raises(ValueError):
        re.relative_l2(p, t[:2])


def test_histogram_cdf_and_streaming():
    torch.manual_seed(1)
    x = torch.randn(1000, 3)
    edges, counts = hist.histogram(x, bins=12)
    assert edges.shape == (13, 3) and counts.shape == (12, 3)
    assert torch.all(counts.sum(0) == 1000)
    for j in range(3):
        ref = torch.histc(x[:, j], bins=12, min=float(x[:, j].min()), max=float(x[:, j].max()))
        assert torch.equal(counts[:, j].float(), ref)
    _, c = hist.cdf(x, bins=12)
    assert torch.allclose(c[-1], torch.ones(3))
    h = hist.Histogram((3,), bins=12)
    h(x[:500])
    h.update(x[500:] * 1.5)
    e2, pdf = h.finalize()
    assert torch.allclose((pdf * (e2[1] - e2[0])).sum(0), torch.ones(3), atol=1e-5)
    assert int(h.counts.sum()) == 3000
    _, cdf2 = h.finalize(cdf=True)
    assert torch.allclose(cdf2[-1], torch.ones(3))
    mids = 0.5 * (edges[1:] + edges[:-1])
    assert torch.allclose(hist.normal_cdf(torch.zeros(3), torch.ones(3), edges),
                          0.5 * (1 + torch.erf(mids / math.sqrt(2))))


def test_crps_forms():
    torch.manual_seed(2)
    ens, obs = torch.randn(200, 7), torch.randn(7)
    k = crps.kcrps(ens, obs, dim=0)
    brute = (ens - obs).abs().mean(0) - 0.5 * (ens[:, None] - ens[None]).abs().mean((0, 1))
    assert torch.allclose(k, brute, atol=1e-5)
    fair = crps.kcrps(ens, obs, dim=0, biased=False)
    brute_fair = (ens - obs).abs().mean(0) - 0.5 * (ens[:, None] - ens[None]).abs().sum((0, 1)) / (200 * 199)
    assert torch.allclose(fair, brute_fair, atol=1e-5)
    big = torch.randn(20000, 2)
    g = crps._crps_gaussian(torch.zeros(2), torch.ones(2), torch.tensor([0.3, -1.0]))
    assert torch.allclose(crps.crps(big, torch.tensor([0.3, -1.0]), method="kernel"), g, atol=2e-2)
    assert torch.allclose(crps.crps(big, torch.tensor([0.3, -1.0]), method="histogram"), g, atol=6e-2)
    with pytest.raises(ValueError):
        crps.crps(big, obs[:2], method="nope")


def test_ensemble_mean_variance_streaming():
    torch.manual_seed(3)
    x = torch.randn(90, 4, 5)
    m, v = em.Mean((4, 5)), em.Variance((4, 5))
    m(x[:30]); v(x[:30])
    for i in (30, 60):
        m.update(x[i:i + 30]); v.update(x[i:i + 30])
    assert torch.allclose(m.finalize(), x.mean(0), atol=1e-6)
    assert torch.allclose(v.finalize(), x.var(0), atol=1e-5)
    assert torch.allclose(v.finalize(std=True), x.std(0), atol=1e-5)
    s, n = em._update_mean(x[:10].sum(0), 10, x[10:20])
    assert n == 20 and torch.allclose(s / n, x[:20].mean(0), atol=1e-6)
    with pytest.raises(ValueError):
        m.update(torch.randn(3, 2, 2))


def test_entropy_wasserstein_calibration():
    torch.manual_seed(4)
    x = torch.randn(50000, 1)
    edges, counts = hist.histogram(x, bins=60)
    ent = entropy.entropy_from_counts(counts.float(), edges, normalized=False)
    assert abs(float(ent) - 0.5 * math.log(2 * math.pi * math.e)) < 3e-2
    assert float(entropy.relative_entropy_from_counts(counts.float(), counts.float(), edges)) < 1e-6
    y = x + 0.5
    assert abs(float(ws.wasserstein_from_samples(x, y, bins=200)) - 0.5) < 5e-2
    w2 = ws.wasserstein_from_normal(torch.zeros(3), torch.eye(3), torch.ones(3), 4 * torch.eye(3))
    assert abs(float(w2) - (3 + 3 * (1 + 4 - 2 * 2))) < 1e-4
    w1 = ws.wasserstein_from_normal(torch.zeros(2), torch.ones(2), torch.ones(2), 4 * torch.ones(2))
    assert torch.allclose(w1, torch.tensor([2.0, 2.0]))
    ranks = torch.rand(5000, 2)
    assert float(calibration.rank_probability_score(ranks).max()) < 1e-2
    r = calibration.find_rank(edges, counts, torch.zeros(1))
    assert abs(float(r) - 0.5) < 5e-2


def test_reductions_and_spectrum():
    torch.manual_seed(5)
    x, w = torch.randn(6, 8), torch.rand(8) + 0.1
    wm = reduction.WeightedMean(w)(x, dim=1)
    assert torch.allclose(wm, (x * w).sum(1) / w.sum(), atol=1e-6)
    wv = reduction.WeightedVariance(w)(x, dim=1)
    ref = ((x - wm[:, None]) ** 2 * w / w.sum()).sum(1) * 8 / 7
    assert torch.allclose(wv, ref, atol=1e-5)
    with pytest.raises(ValueError):
        reduction.WeightedMean(torch.tensor([1.0, -1.0]))
    f = torch.randn(2, 32, 32)
    k, p = ps.power_spectrum(f)
    assert k.shape == (15,) and p.shape == (2, 15)
    assert torch.all(p[torch.isfinite(p)] >= 0)


def test_climate_metrics():
    torch.manual_seed(6)
    lat = torch.linspace(-90, 90, 19)
    x = torch.randn(3, 19, 36)
    w = torch.cos(torch.deg2rad(lat)).abs()
    w = w / w.sum()
    assert torch.allclose(clim_red.global_mean(x, lat), (x * w[:, None]).sum(1).mean(-1), atol=1e-6)
    assert torch.all(clim_red.global_var(x, lat, std=True) > 0)
    assert clim_red.zonal_var(x, lat).shape == (3, 36)
    clim = torch.zeros(3, 19, 36)
    assert torch.allclose(acc_mod.acc(x, x, clim, lat), torch.ones(3), atol=1e-5)
    assert torch.allclose(acc_mod.acc(x, -x, clim, lat), -torch.ones(3), atol=1e-5)
    s = torch.randn(40000, 1)
    edges, counts = hist.histogram(s, bins=50)
    _, c = hist.cdf(s, bins=edges)
    assert abs(float(efi_mod.efi_gaussian(c, edges, torch.zeros(1), torch.ones(1)))) < 2e-2
    shifted = efi_mod.efi_gaussian(hist.cdf(s + 2.0, bins=edges)[1], edges, torch.zeros(1), torch.ones(1))
    assert float(shifted) > 0.5


def test_losses():
    torch.manual_seed(7)
    a = torch.rand(2, 3, 16, 16)
    ssim = SSIM()
    assert abs(float(ssim(a, a)) - 1.0) < 1e-5
    assert float(ssim(a, torch.rand_like(a))) < 0.5

    class _M:
        output_channels, output_time_dim, input_time_dim = 2, 2, 1
        output_variables = ["z500", "tcwv0"]

    p, t = torch.rand(1, 2, 2, 12, 8, 8), torch.rand(1, 2, 2, 12, 8, 8)
    assert float(MSE_SSIM(ssim_params={'time_series_forecasting': True})(p, t, _M())) > 0
    area = torch.rand(5, 6)
    x1 = torch.randn(2, 3, 5, 6, requires_grad=True)
    x2 = x1.detach().clone().requires_grad_(True)
    y = torch.randn(2, 3, 5, 6)
    l1 = CellAreaWeightedLossFunction(area)(x1, y)
    l2 = CustomCellAreaWeightedLossFunction(area)(x2, y)
    l1.backward(); l2.backward()
    assert torch.allclose(l1, l2) and torch.allclose(x1.grad, x2.grad, atol=1e-7)


def test_cae():
    n = np.array([[1.0, 0, 0], [0, 1.0, 0]])
    tot, cp, cf = cfd.compute_force_coefficients(n, np.array([2.0, 1.0]), 0.5, np.array([3.0, 5.0]),
                                                 np.array([[0.1, 0, 0], [0.2, 0, 0]]))
    assert abs(cp - 3.0) < 1e-12 and abs(cf + 0.5 * (0.2 + 0.2)) < 1e-12 and abs(tot - (cp + cf)) < 1e-12
    tt = np.arange(256) * 0.01
    assert abs(cfd.dominant_freq_calc(np.sin(2 * np.pi * 5 * tt), 0.01) - 5.0) < 0.5
    g = torch.randn(2, 3, 3, 4, 4, 4)
    P, Q, R = cfd.compute_p_q_r(g)
    assert P.shape == Q.shape == R.shape == (2, 64)
    fld = np.random.default_rng(0).standard_normal((3, 8, 8, 8))
    mk, E, wn, tke = cfd.compute_tke_spectrum(fld)
    ref = np.zeros(9)
    u = [np.fft.fftn(fld[i]) / 512 for i in range(3)]
    e3 = 0.5 * sum(np.abs(c) ** 2 for c in u)
    for i in range(8):
        for j in range(8):
            for k in range(8):
                r = int(np.round(np.sqrt(i * i + j * j + k * k)))
                if r < 9:
                    ref[r] += e3[i, j, k]
    assert np.allclose(tke, ref) and mk.shape == E.shape == (512,)
    pts = np.array([[0.0, 0, 0], [1, 0, 0], [1, 1, 0]])
    edges = np.array([[0, 1], [1, 2]])
    assert abs(integral.line_integral(edges, pts, np.array([2.0, 3.0])) - 5.0) < 1e-12
    assert abs(integral.line_integral(edges, pts, np.array([[1.0, 0, 0], [1.0, 0, 0]])) - 1.0) < 1e-12
