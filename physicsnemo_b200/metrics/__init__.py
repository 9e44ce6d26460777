"""Metrics: ``general`` (statistics and scores), ``climate`` (lat-weighted, ACC, EFI, losses), ``cae`` (CFD integrals)."""
