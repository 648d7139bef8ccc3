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
