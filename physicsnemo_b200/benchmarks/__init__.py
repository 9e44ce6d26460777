"""Training-throughput benchmarks of the five headline configurations.

Each module exposes ``run(args, rank, world, dev) -> dict`` (the fields of the benchmark's JSON line) and is driven by
``bench.py`` at the repository root: ``transolver`` (1 M-point cloud, points sharded), ``songunet`` (EDM SongUNet 1024²,
height-sharded through ``ShardTensor``), ``mgn`` (MeshGraphNet 2 M nodes, graph partitioned with 1-hop halos), ``afno``
(AFNO 720×1440, token / channel resharding around the spectral filter) and ``fno`` (FNO-2D on the CPU).
All inputs are synthetic and seeded; weights are randomly initialised.
"""
CONFIGS = ("transolver", "songunet", "mgn", "afno", "fno")
