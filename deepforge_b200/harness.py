"""Device-side plumbing for running a Workload through the public Executable interface:
torch is used only as the allocator and copy engine (pinned host buffers, device buffers,
streams); every computation goes through Executable.execute()."""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from . import runtime, synthetic
from .workloads import Workload


class Session:
    def __init__(self, workload: Workload, device: Optional[torch.device] = None, options: int = 0, pin: bool = False):
        self.workload = workload
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.exe = runtime.compile_graph(workload.document, options=options)
        self.host: Dict[int, torch.Tensor] = {}
        self.dev: Dict[int, torch.Tensor] = {}
        for uid, make in workload.inputs.items():
            array = np.ascontiguousarray(make()).reshape(-1).view(np.uint8)
            host = torch.from_numpy(array.copy())
            self.host[uid] = host.pin_memory() if pin else host
            self.dev[uid] = self.host[uid].to(self.device, non_blocking=False)
        for uid, make in workload.device_inputs.items():
            self.dev[uid] = make(self.device).view(torch.uint8).reshape(-1)
        for argument in self.exe.arguments():
            uid = argument["uid"]
            if uid not in self.dev:
                self.dev[uid] = torch.zeros(max(argument["size_bytes"], 1), dtype=torch.uint8, device=self.device)
        size = self.exe.workspace_size
        self.workspace = torch.empty(max(size, 1), dtype=torch.uint8, device=self.device) if size else None
        self.pack = {uid: tensor.data_ptr() for uid, tensor in self.dev.items()}

    @property
    def workspace_ptr(self) -> int:
        return self.workspace.data_ptr() if self.workspace is not None else 0

    def run(self) -> None:
        self.exe.execute(self.pack, self.workspace_ptr)

    # ---- replicas: independent copies of every buffer, so that back-to-back steps touch cold data ----

    def footprint_bytes(self) -> int:
        return sum(t.numel() for t in self.dev.values()) + (self.workspace.numel() if self.workspace is not None else 0)

    def make_replicas(self, count: int) -> None:
        """Replica 0 is the session's own buffers; replicas 1.. are device-side copies (inputs copied,
        outputs and workspace fresh). Read-only tensors above 256 MiB (the paged KV pool) are shared:
        one pass over them already exceeds the L2 several times."""
        self.replicas = [(self.pack, self.workspace_ptr)]
        self._replica_buffers = []
        written = {a["uid"] for a in self.exe.arguments() if a["access"] != "read"}
        for _ in range(1, count):
            buffers = {}
            for uid, tensor in self.dev.items():
                if uid not in written and tensor.numel() > (256 << 20):
                    buffers[uid] = tensor
                else:
                    buffers[uid] = tensor.clone()
            workspace = torch.empty_like(self.workspace) if self.workspace is not None else None
            self._replica_buffers.append((buffers, workspace))
            self.replicas.append(({uid: t.data_ptr() for uid, t in buffers.items()}, workspace.data_ptr() if workspace is not None else 0))

    def capture(self, first: Optional[int] = None, last: Optional[int] = None):
        """One CUDA graph per replica holding plan steps [first, last) (default: the whole plan)."""
        if not hasattr(self, "replicas"):
            self.make_replicas(1)
        stream = torch.cuda.Stream(self.device)
        graphs = []
        lo = 0 if first is None else first
        hi = len(self.exe.steps()) if last is None else last
        with torch.cuda.stream(stream):
            self.exe.set_stream(stream.cuda_stream)
            for pack, workspace in self.replicas:  # warm-up outside capture (one-time kernel attribute calls)
                self.exe.execute_steps(lo, hi, pack, workspace)
            torch.cuda.synchronize(self.device)
            for pack, workspace in self.replicas:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    self.exe.execute_steps(lo, hi, pack, workspace)
                graphs.append(graph)
        self.exe.set_stream(None)
        torch.cuda.synchronize(self.device)
        return graphs

    def capture_round(self, first: int, last: int):
        """ONE CUDA graph holding plan steps [first, last) of every replica in turn: the launches follow one another
        the way they do inside a step (chained, each on buffers the one before did not touch), so a replay measures
        what a launch costs in a stream of launches rather than alone behind a graph launch."""
        if not hasattr(self, "replicas"):
            self.make_replicas(1)
        stream = torch.cuda.Stream(self.device)
        with torch.cuda.stream(stream):
            self.exe.set_stream(stream.cuda_stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for pack, workspace in self.replicas:
                    self.exe.execute_steps(first, last, pack, workspace)
        self.exe.set_stream(None)
        torch.cuda.synchronize(self.device)
        return graph

    def replica_tensors(self, index: int) -> Dict[int, torch.Tensor]:
        return self.dev if index == 0 else self._replica_buffers[index - 1][0]

    def run_pipelined(self, steps: int, graphs, host_outputs) -> None:
        """`steps` end-to-end passes: every pass copies all host-generated inputs from pinned memory to the
        device, replays Executable.execute() and copies all outputs to pinned host memory. The three phases
        run on three streams over the buffer replicas, so that the upload of pass i+1, the kernels of pass i
        and the download of pass i-1 overlap (PCIe carries both directions at once). `graphs` come from
        capture(); `host_outputs[r][uid]` is the pinned destination of replica r. The caller synchronises."""
        count = len(self.replicas)
        if not hasattr(self, "_pipeline"):
            make = lambda: [torch.cuda.Event() for _ in range(count)]
            self._pipeline = (torch.cuda.Stream(self.device), torch.cuda.Stream(self.device), torch.cuda.Stream(self.device), make(), make(), make())
        up, compute, down, uploaded, computed, downloaded = self._pipeline
        start = torch.cuda.Event()
        start.record(torch.cuda.current_stream(self.device))
        for stream in (up, compute, down):
            stream.wait_event(start)
        for i in range(steps):
            r = i % count
            tensors = self.replica_tensors(r)
            with torch.cuda.stream(up):
                if i >= count:
                    up.wait_event(computed[r])  # the kernels of pass i - count have read this replica's inputs
                for uid, host in self.host.items():
                    tensors[uid].copy_(host, non_blocking=True)
                uploaded[r].record(up)
            with torch.cuda.stream(compute):
                compute.wait_event(uploaded[r])
                if i >= count:
                    compute.wait_event(downloaded[r])  # its previous outputs are on the host
                graphs[r].replay()
                computed[r].record(compute)
            with torch.cuda.stream(down):
                down.wait_event(computed[r])
                for uid, host in host_outputs[r].items():
                    host.copy_(tensors[uid], non_blocking=True)
                downloaded[r].record(down)
        main = torch.cuda.current_stream(self.device)
        for r in range(min(count, steps)):
            main.wait_event(downloaded[r])

    def run_steps(self, first: int, last: int) -> None:
        self.exe.execute_steps(first, last, self.pack, self.workspace_ptr)

    def upload(self, stream: Optional[torch.cuda.Stream] = None) -> int:
        """Copy every host-generated input to the device again; returns the bytes moved."""
        moved = 0
        for uid, host in self.host.items():
            self.dev[uid].copy_(host, non_blocking=True)
            moved += host.numel()
        return moved

    def raw(self, uid: int) -> np.ndarray:
        torch.cuda.synchronize(self.device)
        return self.dev[uid].cpu().numpy()

    def output(self, uid: int) -> np.ndarray:
        """Tensor contents widened to f32 (floating types) or as stored integers/codes."""
        data_type = self.workload.tensor(uid)["data_type"]
        raw = self.raw(uid)
        if data_type == "BFLOAT16":
            return synthetic.bf16_bits_to_f32(raw.view(np.uint16))
        if data_type == "FLOAT":
            return raw.view(np.float32).copy()
        if data_type == "HALF":
            return raw.view(np.float16).astype(np.float32)
        if data_type == "INT32":
            return raw.view(np.int32).copy()
        return raw.copy()
