"""Active-learning driver on CPU: full cycle, strategy serialisation, checkpoint resume."""
import json
import queue

import pytest
import torch

from physicsnemo_b200.active_learning import (DefaultTrainingLoop, Driver, DriverConfig, OptimizerConfig,
                                              StrategiesConfig, TrainingConfig, registry)
from physicsnemo_b200.active_learning import protocols as p
from physicsnemo_b200.active_learning.logger import log_context, setup_active_learning_logger
from physicsnemo_b200.models.mlp import FullyConnected


class ListQueue:
    def __init__(self):
        self.items = []

    def put(self, item):
        self.items.append(item)

    def get(self):
        return self.items.pop(0)

    def empty(self):
        return not self.items

    def to_list(self):
        return list(self.items)

    def from_list(self, items):
        self.items = list(items)


class Pool(torch.utils.data.Dataset):
    def __init__(self, n):
        g = torch.Generator().manual_seed(0)
        self.rows = [(x, (2 * x).sum(0, keepdim=True)) for x in torch.randn(n, 3, generator=g)]

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        return self.rows[i]

    def append(self, item):
        self.rows.append(item)


class FarthestQuery(p.QueryStrategy):
    def __init__(self, max_samples: int = 4, scale: float = 3.0):
        self.max_samples, self.scale = max_samples, scale

    def sample(self, query_queue, *a, **k):
        for i in range(self.max_samples):
            query_queue.put(torch.full((3,), self.scale * (i + 1)))


class ExactLabel(p.LabelStrategy):
    __is_external_process__ = False

    def __init__(self):
        pass

    def label(self, queue_to_label, serialize_queue, *a, **k):
        while not queue_to_label.empty():
            x = queue_to_label.get()
            serialize_queue.put((x, (2 * x).sum(0, keepdim=True)))


class CountMetric(p.MetrologyStrategy):
    def __init__(self, tag: str = "m"):
        self.tag, self.records = tag, []

    def compute(self, *a, **k):
        self.append({"step": self.driver.active_learning_step_idx, "pool": len(self.driver.train_datapool)})

    def serialize_records(self, path=None, *a, **k):
        (self.strategy_dir / "records.json").write_text(json.dumps(self.records))


def _train_step(model, batch):
    x, y = batch
    return torch.nn.functional.mse_loss(model(x), y)


def _driver(tmp_path, **cfg):
    model = FullyConnected(in_features=3, layer_size=8, out_features=1, num_layers=1)
    loop = DefaultTrainingLoop(train_step_fn=_train_step, enable_static_capture=False, use_progress_bars=False)
    tc = TrainingConfig(train_datapool=Pool(16), max_training_epochs=2, max_fine_tuning_epochs=1,
                        optimizer_config=OptimizerConfig(torch.optim.SGD, {"lr": 1e-2}), train_loop_fn=loop)
    sc = StrategiesConfig(query_strategies=[FarthestQuery(max_samples=3)], queue_cls=ListQueue,
                          label_strategy=ExactLabel(), metrology_strategies=[CountMetric(tag="a")])
    dc = DriverConfig(batch_size=8, max_active_learning_steps=2, root_log_dir=tmp_path, device="cpu", **cfg)
    return Driver(dc, model, sc, tc)


def test_full_cycle_and_resume(tmp_path):
    d = _driver(tmp_path)
    before = [w.clone() for w in d.learner.parameters()]
    d.run()
    assert d.active_learning_step_idx == 2 and len(d.train_datapool) == 16 + 2 * 3
    assert any(not torch.equal(a, b) for a, b in zip(before, d.learner.parameters()))
    metric = d.metrology_strategies[0]
    assert [r["pool"] for r in metric.records] == [16, 19] and (metric.strategy_dir / "records.json").exists()
    log_lines = (d.log_dir / f"{d.run_id}.log").read_text().strip().splitlines()
    assert any(json.loads(line).get("phase") == "labeling" for line in log_lines)
    # the labeling checkpoint of step 1 was taken with the query queue filled
    ckpt = d.log_dir / "checkpoints" / "step_1" / "labeling"
    assert (ckpt / "checkpoint.pt").exists() and (ckpt / "FullyConnected.mdlus").exists()
    r = Driver.load_checkpoint(ckpt, train_datapool=Pool(16),
                               driver_config_overrides={"root_log_dir": tmp_path / "resume"})
    assert r.active_learning_step_idx == 1 and str(r.current_phase) == "labeling"
    assert len(r.query_queue.items) == 3 and isinstance(r.query_strategies[0], FarthestQuery)
    assert r.query_strategies[0].max_samples == 3 and r.metrology_strategies[0].tag == "a"
    r.active_learning_step()                      # runs only the labeling phase of step 1
    assert len(r.train_datapool) == 19 and r.active_learning_step_idx == 2 and r.current_phase is None


def test_configs_validate_and_roundtrip(tmp_path):
    with pytest.raises(ValueError):
        OptimizerConfig(optimizer_kwargs={"lr": -1})
    with pytest.raises(ValueError):
        OptimizerConfig(scheduler_kwargs={"gamma": 0.1})
    with pytest.raises(ValueError):
        StrategiesConfig(query_strategies=[], queue_cls=queue.Queue)
    with pytest.raises(ValueError):
        DriverConfig(batch_size=0)
    oc = OptimizerConfig(torch.optim.Adam, {"lr": 1e-3}, torch.optim.lr_scheduler.StepLR, {"step_size": 2})
    back = OptimizerConfig.from_dict(oc.to_dict())
    assert back.optimizer_cls is torch.optim.Adam and back.scheduler_cls is torch.optim.lr_scheduler.StepLR
    dc = DriverConfig(batch_size=4, root_log_dir=tmp_path, dtype=torch.float64, device="cpu")
    again = DriverConfig.from_json(dc.to_json())
    assert again.batch_size == 4 and again.dtype is torch.float64 and again.run_id == dc.run_id
    assert again.max_active_learning_steps == float("inf")
    loop = DefaultTrainingLoop(enable_static_capture=False, device=torch.device("cpu"), dtype=torch.float32)
    assert loop._args["__args__"]["device"] == "cpu" and loop._args["__args__"]["dtype"] == "torch.float32"
    with pytest.raises(ValueError):
        _driver(tmp_path, skip_training=True, fine_tuning_lr=1e-3)


def test_registry_and_logger(tmp_path):
    name = "FarthestQueryForTest"
    if not registry.is_registered(name):
        registry.register(name)(FarthestQuery)
    with pytest.raises(ValueError):
        registry.register(name)(FarthestQuery)
    q = registry.construct(name, max_samples=2)
    assert q.max_samples == 2 and q._args["__args__"] == {"max_samples": 2, "scale": 3.0}
    with pytest.warns(UserWarning), pytest.raises(TypeError):
        registry.construct(name, bogus=1)
    with pytest.raises(NameError):
        registry.get_class("Nope")
    assert registry.get_class("SGD", "torch.optim") is torch.optim.SGD
    with pytest.raises(RuntimeError):
        _ = FarthestQuery().strategy_dir
    log = setup_active_learning_logger("al.test", "rid", tmp_path)
    with log_context(caller_object="Q", iteration=3, phase="query", budget=5):
        log.info("hello")
    entry = json.loads((tmp_path / "rid.log").read_text().strip().splitlines()[-1])
    assert entry["message"] == "hello" and entry["iteration"] == 3 and entry["context"] == {"budget": 5}
