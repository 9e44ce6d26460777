"""``DistributedManager``: one process per GPU, rank / device / group bookkeeping.

Parity: ``physicsnemo/distributed/manager.py`` — shared-state singleton (``:66-126``),
properties (``:133-293``), ``initialize`` over ENV → SLURM → OpenMPI with the override
``PHYSICSNEMO_DISTRIBUTED_INITIALIZATION_METHOD`` (``:371-435``), ``initialize_mesh``
(``:437-521``), ``get_mesh_group`` (``:524-554``), ``setup`` (``:556-610``), sub-group helpers
(``:612-799``), ``cleanup`` (``:801-824``).

Beyond the reference, the manager owns the peer-memory runtime of this framework
(``peer_runtime()``): symmetric buffers and signal pads used by the in-kernel collectives.
"""
from __future__ import annotations

import atexit
import os
import queue
import warnings
from typing import Optional, Tuple
from warnings import warn

import numpy as np
import torch
import torch.distributed as dist

from .config import ProcessGroupConfig, ProcessGroupNode


class PhysicsNeMoUndefinedGroupError(Exception):
    """Raised when a process group is requested that was never created."""

    def __init__(self, name: str):
        super().__init__(f"Cannot query process group '{name}' before it is explicitly created.")


class PhysicsNeMoUninitializedDistributedManagerWarning(Warning):
    """Issued when the manager is instantiated before ``initialize()``."""

    def __init__(self):
        super().__init__(
            "A DistributedManager object is being instantiated before "
            "this singleton class has been initialized. Instantiating a manager before "
            "initialization can lead to unexpected results where processes fail "
            "to communicate. Initialize the distributed manager via "
            "DistributedManager.initialize() before instantiating."
        )


class DistributedManager:
    """Process-wide view of the distributed job (shared state across instances)."""

    _shared_state: dict = {}

    def __new__(cls):
        obj = super().__new__(cls)
        obj.__dict__ = cls._shared_state
        defaults = dict(
            _rank=0, _world_size=1, _local_rank=0, _distributed=False,
            _device=torch.device("cuda:0" if torch.cuda.is_available() else "cpu"),
            _cuda=torch.cuda.is_available(), _broadcast_buffers=False, _find_unused_parameters=False,
            _initialization_method="None", _groups={}, _group_ranks={}, _group_names={}, _is_initialized=False,
            _global_mesh=None, _mesh_groups={}, _peer_runtime=None,
        )
        for k, v in defaults.items():
            if not hasattr(obj, k):
                setattr(obj, k, v)
        return obj

    def __init__(self):
        if not self._is_initialized:
            raise PhysicsNeMoUninitializedDistributedManagerWarning()
        super().__init__()

    # ------------------------------------------------------------ properties
    @property
    def rank(self):
        return self._rank

    @property
    def local_rank(self):
        return self._local_rank

    @property
    def world_size(self):
        return self._world_size

    @property
    def device(self):
        return self._device

    @property
    def distributed(self):
        return self._distributed

    @property
    def cuda(self):
        return self._cuda

    @property
    def mesh_dims(self):
        return () if self._global_mesh is None else tuple(self._global_mesh.mesh_dim_names)

    @property
    def group_names(self):
        return self._groups.keys()

    @property
    def global_mesh(self):
        if self._global_mesh is None:
            self.initialize_mesh(mesh_shape=(-1,), mesh_dim_names=("world",))
        return self._global_mesh

    def mesh(self, name=None):
        """Mesh named ``name`` (a sub-mesh of the global mesh) or the global mesh."""
        if name is None:
            return self.global_mesh
        return self.global_mesh[name]

    def group(self, name=None):
        if name in self._groups:
            return self._groups[name]
        if name is None:
            return None
        raise PhysicsNeMoUndefinedGroupError(name)

    def group_size(self, name=None):
        if name is None:
            return self._world_size
        return dist.get_world_size(group=self.group(name))

    def group_rank(self, name=None):
        if name is None:
            return self._rank
        return dist.get_rank(group=self.group(name))

    def group_name(self, group=None):
        if group is None:
            return None
        return self._group_names[group]

    @property
    def broadcast_buffers(self):
        return self._broadcast_buffers

    @broadcast_buffers.setter
    def broadcast_buffers(self, value: bool):
        self._broadcast_buffers = value

    @property
    def find_unused_parameters(self):
        return self._find_unused_parameters

    @find_unused_parameters.setter
    def find_unused_parameters(self, value: bool):
        if value:
            warn("Setting `find_unused_parameters` in DDP to true, use only if necessary.")
        self._find_unused_parameters = value

    def __str__(self):
        return (
            f"Initialized process {self.rank} of {self.world_size} using method "
            f"'{self._initialization_method}'. Device set to {str(self.device)}"
        )

    @classmethod
    def is_initialized(cls) -> bool:
        return cls._shared_state.get("_is_initialized", False)

    # ---------------------------------------------------------- bring-up
    @staticmethod
    def get_available_backend():
        if torch.cuda.is_available() and dist.is_nccl_available():
            return "nccl"
        return "gloo"

    @staticmethod
    def _local_rank_default(rank):
        n = torch.cuda.device_count()
        return rank % n if n > 0 else 0

    @staticmethod
    def initialize_env():
        rank = int(os.environ.get("RANK"))  # TypeError when unset -> caller falls through
        world_size = int(os.environ.get("WORLD_SIZE"))
        local_rank = os.environ.get("LOCAL_RANK")
        local_rank = int(local_rank) if local_rank is not None else DistributedManager._local_rank_default(rank)
        DistributedManager.setup(
            rank=rank, world_size=world_size, local_rank=local_rank, addr=os.environ.get("MASTER_ADDR"),
            port=os.environ.get("MASTER_PORT"), backend=DistributedManager.get_available_backend(),
        )

    @staticmethod
    def initialize_open_mpi(addr, port):
        rank = int(os.environ.get("OMPI_COMM_WORLD_RANK"))
        world_size = int(os.environ.get("OMPI_COMM_WORLD_SIZE"))
        local_rank = int(os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK"))
        DistributedManager.setup(rank=rank, world_size=world_size, local_rank=local_rank, addr=addr, port=port,
                                 backend=DistributedManager.get_available_backend(), method="openmpi")

    @staticmethod
    def initialize_slurm(port):
        rank = int(os.environ.get("SLURM_PROCID"))
        world_size = int(os.environ.get("SLURM_NPROCS"))
        local_rank = int(os.environ.get("SLURM_LOCALID"))
        addr = os.environ.get("SLURM_LAUNCH_NODE_IPADDR")
        DistributedManager.setup(rank=rank, world_size=world_size, local_rank=local_rank, addr=addr, port=port,
                                 backend=DistributedManager.get_available_backend(), method="slurm")

    @staticmethod
    def initialize():
        """Initialise from the launcher environment (ENV, then SLURM, then OpenMPI)."""
        if DistributedManager.is_initialized():
            warn("Distributed manager is already initialized")
            return
        addr = os.getenv("MASTER_ADDR", "localhost")
        port = os.getenv("MASTER_PORT", "12355")
        os.environ["TORCH_NCCL_ASYNC_ERROR_HANDLING"] = "0"
        method = os.getenv("PHYSICSNEMO_DISTRIBUTED_INITIALIZATION_METHOD")
        if method is None:
            try:
                DistributedManager.initialize_env()
            except TypeError:
                if "SLURM_PROCID" in os.environ:
                    DistributedManager.initialize_slurm(port)
                elif "OMPI_COMM_WORLD_RANK" in os.environ:
                    DistributedManager.initialize_open_mpi(addr, port)
                else:
                    warn("Could not initialize using ENV, SLURM or OPENMPI methods. Assuming this is a single process job")
                    DistributedManager._shared_state["_is_initialized"] = True
        elif method == "ENV":
            DistributedManager.initialize_env()
        elif method == "SLURM":
            DistributedManager.initialize_slurm(port)
        elif method == "OPENMPI":
            DistributedManager.initialize_open_mpi(addr, port)
        else:
            raise RuntimeError(
                f"Unknown initialization method {method}. Supported values for "
                "PHYSICSNEMO_DISTRIBUTED_INITIALIZATION_METHOD are ENV, SLURM and OPENMPI"
            )
        np.random.seed(seed=DistributedManager().rank)

    @staticmethod
    def setup(rank=0, world_size=1, local_rank=None, addr="localhost", port="12355", backend="nccl", method="env"):
        """Create the default process group and record rank / device."""
        os.environ["MASTER_ADDR"] = addr or "localhost"
        os.environ["MASTER_PORT"] = str(port or "12355")
        DistributedManager._shared_state["_is_initialized"] = True
        m = DistributedManager()
        m._distributed = dist.is_available()
        if m._distributed:
            m._rank, m._world_size = rank, world_size
            m._local_rank = DistributedManager._local_rank_default(rank) if local_rank is None else local_rank
        m._device = torch.device(f"cuda:{m.local_rank}" if torch.cuda.is_available() else "cpu")
        if m._distributed and not dist.is_initialized():
            kwargs = dict(rank=m.rank, world_size=m.world_size)
            if m._device.type == "cuda":
                kwargs["device_id"] = m._device
            dist.init_process_group(backend, **kwargs)
        if torch.cuda.is_available():
            torch.cuda.set_device(m.device)
            torch.cuda.empty_cache()
        m._initialization_method = method
        atexit.register(DistributedManager.cleanup)

    # ---------------------------------------------------------------- meshes
    def initialize_mesh(self, mesh_shape: Tuple[int, ...], mesh_dim_names: Tuple[str, ...]):
        """Create the global ``DeviceMesh``; one entry of ``mesh_shape`` may be ``-1``."""
        if self._global_mesh is not None:
            raise RuntimeError("Global mesh already initialized; it can only be created once")
        if not self._distributed or not dist.is_initialized():
            raise RuntimeError("initialize_mesh requires an initialized process group")
        mesh_shape = list(mesh_shape)
        if len(mesh_shape) != len(mesh_dim_names):
            raise RuntimeError("Device mesh shape and dimension names must have the same length")
        if mesh_shape.count(-1) > 1:
            raise RuntimeError("At most one mesh dimension may be -1")
        if -1 in mesh_shape:
            known = int(np.prod([s for s in mesh_shape if s != -1]))
            if self.world_size % known:
                raise RuntimeError(f"World size {self.world_size} is not divisible by the fixed mesh dims {known}")
            mesh_shape[mesh_shape.index(-1)] = self.world_size // known
        if int(np.prod(mesh_shape)) != self.world_size:
            raise RuntimeError(f"Device mesh size {tuple(mesh_shape)} does not match world size {self.world_size}")
        self._global_mesh = dist.init_device_mesh(self.device.type, tuple(mesh_shape), mesh_dim_names=tuple(mesh_dim_names))
        for name in mesh_dim_names:
            grp = self._global_mesh[name].get_group()
            self._groups[name] = grp
            self._group_names[grp] = name
        return self._global_mesh

    def get_mesh_group(self, mesh) -> Optional[dist.ProcessGroup]:
        """Process group covering every rank of ``mesh`` (flattening N-D meshes, cached)."""
        if mesh.ndim == 1:
            return mesh.get_group()
        ranks = tuple(mesh.mesh.flatten().tolist())
        if ranks in self._mesh_groups:
            return self._mesh_groups[ranks]
        # every rank must take part in every new_group call: build one group per flattened slice
        parent = self._global_mesh if self._global_mesh is not None else mesh
        all_ranks = parent.mesh.flatten().tolist()
        grp = dist.new_group(ranks=list(ranks), use_local_synchronization=True) if set(ranks) <= set(all_ranks) else None
        self._mesh_groups[ranks] = grp
        return grp

    # ------------------------------------------------------ legacy sub-groups
    @staticmethod
    def create_process_subgroup(name: str, size: int, group_name: Optional[str] = None, verbose: bool = False):
        """Split ``group_name`` (default: world) into consecutive groups of ``size`` ranks."""
        m = DistributedManager()
        if not m.distributed:
            raise AssertionError("torch.distributed is unavailable. Check pytorch build to ensure the distributed package is available.")
        if name in m._groups:
            raise AssertionError(f"Group with name {name} already exists")
        group = m._groups.get(group_name) if group_name else None
        group_size = dist.get_world_size(group=group)
        if group_size % size:
            raise AssertionError(f"Cannot divide group size {group_size} evenly into subgroups of size {size}")
        parent_ranks = m._group_ranks[group_name] if group_name else [list(range(m.world_size))]
        m._group_ranks[name] = []
        for ranks in parent_ranks:
            for i in range(len(ranks) // size):
                sub = ranks[i * size:(i + 1) * size]
                m._group_ranks[name].append(sub)
                tmp = dist.new_group(ranks=sub)
                if m.rank in sub:
                    m._groups[name] = tmp
                    m._group_names[tmp] = name
        if verbose and m.rank == 0:
            print(f"Process group '{name}':")
            for g in m._group_ranks[name]:
                print("    ", g)

    @staticmethod
    def create_orthogonal_process_group(orthogonal_group_name: str, group_name: str, verbose: bool = False):
        """Groups that take the i-th member of every ``group_name`` group."""
        m = DistributedManager()
        if not m.distributed:
            raise AssertionError("torch.distributed is unavailable. Check pytorch build to ensure the distributed package is available.")
        if group_name not in m._groups:
            raise ValueError(f"Group with name {group_name} does not exist")
        if orthogonal_group_name in m._groups:
            raise ValueError(f"Group with name {orthogonal_group_name} already exists")
        ortho = [list(t) for t in zip(*m._group_ranks[group_name])]
        m._group_ranks[orthogonal_group_name] = ortho
        for ranks in ortho:
            tmp = dist.new_group(ranks=ranks)
            if m.rank in ranks:
                m._groups[orthogonal_group_name] = tmp
                m._group_names[tmp] = orthogonal_group_name
        if verbose and m.rank == 0:
            print(f"Process group '{orthogonal_group_name}':")
            for g in ortho:
                print("    ", g)

    @staticmethod
    def create_group_from_node(node: ProcessGroupNode, parent: Optional[str] = None, verbose: bool = False):
        if node.size is None:
            raise AssertionError("Cannot create groups from a ProcessGroupNode that is not fully populated.")
        DistributedManager.create_process_subgroup(node.name, node.size, group_name=parent, verbose=verbose)
        orthogonal = f"__orthogonal_to_{node.name}"
        DistributedManager.create_orthogonal_process_group(orthogonal, node.name, verbose=verbose)
        return orthogonal

    @staticmethod
    def create_groups_from_config(config: ProcessGroupConfig, verbose: bool = False):
        """Breadth-first creation of the named groups of a ``ProcessGroupConfig`` tree."""
        q = queue.Queue()
        q.put(config.root_id)
        DistributedManager.create_group_from_node(config.root)
        while not q.empty():
            node_id = q.get()
            if verbose:
                print(f"Node ID: {node_id}")
            children = config.tree.children(node_id)
            if verbose:
                print(f"  Children: {children}")
            parent_group = node_id
            for child in children:
                parent = DistributedManager.create_group_from_node(child.data, parent=parent_group, verbose=verbose)
                q.put(child.identifier)
                parent_group = parent

    # ---------------------------------------------------------- peer runtime
    def peer_runtime(self, group=None):
        """The peer-memory runtime (symmetric buffers, signal pads) for ``group`` (lazy)."""
        from ..parallel.peer import PeerRuntime

        key = id(group) if group is not None else None
        if self._peer_runtime is None:
            self._peer_runtime = {}
        if key not in self._peer_runtime:
            self._peer_runtime[key] = PeerRuntime(group)
        return self._peer_runtime[key]

    # --------------------------------------------------------------- teardown
    @staticmethod
    def cleanup(barrier: bool = False):
        """Destroy the process group (registered with ``atexit``) and reset the shared state."""
        state = DistributedManager._shared_state
        try:
            if state.get("_distributed") and dist.is_available() and dist.is_initialized():
                if barrier:
                    if state.get("_device") is not None and state["_device"].type == "cuda":
                        dist.barrier(device_ids=[state["_local_rank"]])
                    else:
                        dist.barrier()
                dist.destroy_process_group()
        except Exception:  # interpreter shutdown: best effort
            pass
        state.clear()
