"""Dataset fed by a sampling server during online RL (REINFORCE-style post-training)
(megatron/data/online_dataset.py:27-131).

Protocol (one TCP connection per refill): the client sends the split name, the server answers with a pickled
list of ``{"prefix": [ids], "completions": [[ids], ...], "rewards": [floats]}`` and closes.  Rewards are
centred either leave-one-out within the group of completions or against a moving average of the last 100
group means.  Only connect to servers you run yourself: the payload is unpickled.
"""
from __future__ import annotations

import pickle
import socket
from typing import List, Union

import numpy as np
import torch


class OnlineDataset(torch.utils.data.Dataset):
    def __init__(self, num_samples, seq_length, leave_one_out=False, data_split="train", name=None,
                 dataserver_ips: Union[str, List[str]] = "localhost",
                 dataserver_ports: Union[int, List[int]] = 10000, timeout_s: float = 600.0):
        from .. import parallel as mpu
        self.num_samples, self.seq_length = num_samples, seq_length
        self.global_rank = mpu.get_data_parallel_rank()
        self.leave_one_out = leave_one_out
        self.data_split = data_split if name is None else name
        self.dataserver_ips, self.dataserver_ports = dataserver_ips, dataserver_ports
        self.timeout_s = timeout_s
        self.reward_buffer: List[float] = []
        self.online_batching_data: List[list] = []

    def __len__(self):
        return self.num_samples         # nominal: the server decides how much data exists

    def _endpoint(self):
        ip = self.dataserver_ips if isinstance(self.dataserver_ips, str) else self.dataserver_ips[self.global_rank]
        port = self.dataserver_ports if isinstance(self.dataserver_ports, int) \
            else self.dataserver_ports[self.global_rank]
        return ip, port

    def centre_rewards(self, rewards):
        r = np.asarray(rewards, dtype=np.float64)
        if self.leave_one_out:
            if len(r) < 2:
                return r.tolist()
            return (r - (r.sum() - r) / (len(r) - 1)).tolist()
        base = float(np.mean(self.reward_buffer)) if self.reward_buffer else 0.0
        self.reward_buffer.append(float(r.mean()))
        del self.reward_buffer[:-100]
        return (r - base).tolist()

    def update_online_batches(self):
        ip, port = self._endpoint()
        print(f"Connecting to {ip}:{port}")
        with socket.create_connection((ip, port), timeout=self.timeout_s) as s:
            s.sendall(self.data_split.encode())
            chunks = []
            while True:
                c = s.recv(1 << 16)
                if not c:
                    break
                chunks.append(c)
        groups = pickle.loads(b"".join(chunks))
        print(f"Received {len(groups)} samples from the server.")
        for g in groups:
            centred = self.centre_rewards(g["rewards"])
            for comp, r, raw in zip(g["completions"], centred, g["rewards"]):
                self.online_batching_data.append([g["prefix"], comp, r, raw])

    def __getitem__(self, idx):
        if not self.online_batching_data:
            self.update_online_batches()
        prefix, comp, reward, raw = self.online_batching_data.pop(0)
        text = list(prefix) + list(comp)
        label = [-100] * len(prefix) + list(comp)
        n = self.seq_length + 1
        text = (text + [0] * n)[:n] if len(text) <= self.seq_length else text
        label = (label + [-100] * n)[:n] if len(label) <= self.seq_length else label
        return {"text": np.array(text, dtype=np.int64), "label": np.array(label, dtype=np.int64),
                "reward": np.array([reward], dtype=np.float32), "raw_reward": np.array([raw], dtype=np.float32)}
