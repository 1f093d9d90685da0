"""Launch renderers: turn a resolved training specification into an inspectable ``LaunchPlan``
(argv + environment + provenance) for ``torch.distributed.run``.

* ``SpeedrunBackend``: one data-parallel mesh (ZeRO-1 Muon / AdamW); the nanochat speedrun entry.
* ``MeshBackend``: tensor / sequence / pipeline / context / expert parallel mesh whose collectives
  are fused into the kernels over peer memory (the role Megatron plays in the reference:
  src/archlab/megatron/backend.py:19-120, src/archlab/launch.py:11-57).

Rendering never touches the GPUs or the network; the plan can be committed, diffed and replayed.
"""
from __future__ import annotations

from dataclasses import dataclass

from ..contracts.launch import LaunchPlan


@dataclass(frozen=True)
class Topology:
    nodes: int = 1
    gpus_per_node: int = 8
    node_rank: str = "env:NODE_RANK"
    master_addr: str = "127.0.0.1"
    master_port: int = 29500

    @property
    def world(self) -> int:
        return self.nodes * self.gpus_per_node


def _torchrun(topology: Topology) -> list[str]:
    argv = ["python", "-m", "torch.distributed.run", f"--nnodes={topology.nodes}",
            f"--nproc-per-node={topology.gpus_per_node}", "--master-addr", topology.master_addr,
            "--master-port", str(topology.master_port)]
    if topology.nodes > 1:
        argv += ["--node-rank", topology.node_rank]
    return argv


_BASE_ENV = {"NCCL_NVLS_ENABLE": "1", "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1", "CUDA_DEVICE_MAX_CONNECTIONS": "8"}


class SpeedrunBackend:
    name = "speedrun"

    def render(self, *, depth: int = 20, device_batch_size: int = 16, total_batch_size: int = 524288,
               max_seq_len: int = 2048, num_iterations: int = -1, run_dir: str = "env:ARCHLAB_RUN_DIR",
               topology: Topology = Topology(), extra: dict | None = None, zero_impl: str = "auto") -> LaunchPlan:
        per_step = device_batch_size * max_seq_len * topology.world
        if total_batch_size % per_step:
            raise ValueError("total batch must be a multiple of device batch x sequence x world size")
        argv = _torchrun(topology) + ["-m", "archlab_b200.train.base_train", f"--depth={depth}",
                                      f"--device-batch-size={device_batch_size}", f"--total-batch-size={total_batch_size}",
                                      f"--max-seq-len={max_seq_len}", f"--num-iterations={num_iterations}",
                                      f"--zero-impl={zero_impl}", "--run-dir", run_dir]
        for k, v in sorted((extra or {}).items()):
            argv.append(f"--{k.replace('_', '-')}={v}")
        meta = {"world_size": topology.world, "grad_accum_steps": total_batch_size // per_step,
                "parallelism": f"dp{topology.world}", "collectives": "peer-memory fused ZeRO-1"}
        return LaunchPlan(self.name, tuple(argv), dict(_BASE_ENV), meta)


class MeshBackend:
    name = "megatron"

    def render(self, *, model: str, tp: int = 1, pp: int = 1, cp: int = 1, ep: int = 1, sequence_parallel: bool = True,
               micro_batch: int = 1, global_batch: int = 128, seq_len: int = 8192, precision: str = "bf16",
               run_dir: str = "env:ARCHLAB_RUN_DIR", topology: Topology = Topology(), extra: dict | None = None) -> LaunchPlan:
        world = topology.world
        model_parallel = tp * pp * cp
        if world % model_parallel:
            raise ValueError("world size must be divisible by tp x pp x cp")
        dp = world // model_parallel
        if ep > 1 and (dp * cp) % ep:
            raise ValueError("expert parallel size must divide the data x context parallel ranks")
        if sequence_parallel and tp == 1:
            sequence_parallel = False
        if global_batch % (micro_batch * dp):
            raise ValueError("global batch must be a multiple of micro batch x data parallel size")
        if precision not in ("bf16", "fp8_block", "fp8_tensor", "nvfp4"):
            raise ValueError("precision must be bf16, fp8_block, fp8_tensor or nvfp4")
        argv = _torchrun(topology) + ["-m", "archlab_b200.train.mesh_train", f"--model={model}", f"--tp={tp}", f"--pp={pp}",
                                      f"--cp={cp}", f"--ep={ep}", f"--micro-batch={micro_batch}",
                                      f"--global-batch={global_batch}", f"--seq-len={seq_len}", f"--precision={precision}",
                                      "--run-dir", run_dir]
        if sequence_parallel:
            argv.append("--sequence-parallel")
        for k, v in sorted((extra or {}).items()):
            argv.append(f"--{k.replace('_', '-')}={v}")
        meta = {"world_size": world, "data_parallel": dp, "grad_accum_steps": global_batch // (micro_batch * dp),
                "parallelism": f"tp{tp}{'+sp' if sequence_parallel else ''} pp{pp} cp{cp} ep{ep} dp{dp}",
                "collectives": "all-gather->GEMM / GEMM->reduce-scatter fused over peer memory; pipeline p2p on NCCL"}
        return LaunchPlan(self.name, tuple(argv), dict(_BASE_ENV), meta)
