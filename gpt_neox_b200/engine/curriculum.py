"""Sequence-length curriculum (the scheduler the reference takes from its engine library,
megatron/training.py:1215-1218; config key ``curriculum_learning``).

    {"enabled": true, "curriculum_type": "seqlen", "min_difficulty": 64, "max_difficulty": 2048,
     "schedule_type": "fixed_linear" | "fixed_root" | "fixed_discrete",
     "schedule_config": {"total_curriculum_step": N, "difficulty_step": 8, "root_degree": 2}
                      | {"difficulty": [..], "max_step": [..]}}
"""
from __future__ import annotations

import math


class CurriculumScheduler:
    def __init__(self, config: dict):
        self.state = {}
        for k in ("min_difficulty", "max_difficulty", "schedule_type"):
            assert k in config, f"Curriculum learning requires the config '{k}'"
        self.state["min_difficulty"] = int(config["min_difficulty"])
        self.state["max_difficulty"] = int(config["max_difficulty"])
        self.state["current_difficulty"] = int(config["min_difficulty"])
        self.state["schedule_type"] = st = config["schedule_type"]
        sc = dict(config.get("schedule_config", {}))
        if st == "fixed_discrete":
            assert "difficulty" in sc and "max_step" in sc, "fixed_discrete needs 'difficulty' and 'max_step'"
            assert len(sc["max_step"]) > 0 and len(sc["difficulty"]) == len(sc["max_step"]) + 1
        elif st in ("fixed_root", "fixed_linear"):
            assert "total_curriculum_step" in sc and "difficulty_step" in sc
            if st == "fixed_root":
                assert "root_degree" in sc
            if sc["difficulty_step"] % 8 != 0:
                print("curriculum: difficulty_step is not a multiple of 8; tensor-core tiles prefer multiples of 8")
        else:
            raise RuntimeError(f"Unsupported curriculum schedule type {st}")
        self.state["schedule"] = sc
        self.first_step = True

    def get_current_difficulty(self):
        return self.state["current_difficulty"]

    def set_current_difficulty(self, difficulty):
        self.state["current_difficulty"] = difficulty

    def get_state(self):
        return self.state

    def set_state(self, state):
        self.state = state

    def _root(self, step, degree):
        s = self.state["schedule"]
        lo, hi = self.state["min_difficulty"], self.state["max_difficulty"]
        frac = (float(step) / s["total_curriculum_step"]) ** (1.0 / degree)
        d = math.floor(frac * (hi - lo) + lo)
        d -= d % s["difficulty_step"]
        return max(lo, min(d, hi)) if d >= lo else lo

    def get_difficulty(self, global_steps):
        st, s = self.state["schedule_type"], self.state["schedule"]
        if st == "fixed_discrete":
            for d, m in zip(s["difficulty"], s["max_step"]):
                if global_steps <= m:
                    return d
            return s["difficulty"][-1]
        return self._root(global_steps, 1 if st == "fixed_linear" else s["root_degree"])

    def update_difficulty(self, global_steps):
        if self.state["current_difficulty"] < self.state["max_difficulty"]:
            self.state["current_difficulty"] = self.get_difficulty(global_steps)
        return self.state["current_difficulty"]
