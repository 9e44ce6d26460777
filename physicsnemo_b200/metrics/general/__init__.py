"""General-purpose metrics (errors, CRPS, calibration, histograms, entropy, Wasserstein, spectra)."""
