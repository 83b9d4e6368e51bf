"""Process launcher: one process per GPU, locally or fanned out over a host file.

Stands where the reference hands its argv to ``deepspeed.launcher.runner.main`` (deepy.py:22-37): same
flags (``--hostfile --include --exclude --num_nodes --num_gpus --master_addr --master_port --launcher
--force_multi --no_ssh_check``), followed by the user script and its arguments.

* one node: the ranks are spawned here as children with RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR /
  MASTER_PORT set; the first child that fails ends the others (exact PIDs) and its exit code is returned.
* several nodes: one command line per host is built for the chosen fan-out tool (pdsh, openmpi, mvapich,
  slurm) that re-enters this module with ``--node_rank``; ``--dry_run`` prints the command instead of
  running it.

Host file format: ``hostname slots=N`` per line; ``--include`` / ``--exclude`` take
``host1:0,1@host2`` (devices optional).
"""
from __future__ import annotations

import argparse
import os
import shlex
import signal
import subprocess
import sys
import time
from collections import OrderedDict

EXPORT_ENVS = ["NCCL", "PYTHON", "MV2", "UCX", "NEOX", "CUDA_DEVICE_MAX_CONNECTIONS"]


def parse_args(argv):
    p = argparse.ArgumentParser(description="gpt-neox-b200 launcher")
    p.add_argument("--hostfile", "-H", type=str, default="/job/hostfile")
    p.add_argument("--include", "-i", type=str, default="")
    p.add_argument("--exclude", "-e", type=str, default="")
    p.add_argument("--num_nodes", type=int, default=-1)
    p.add_argument("--num_gpus", type=int, default=-1)
    p.add_argument("--master_port", type=int, default=29500)
    p.add_argument("--master_addr", type=str, default="")
    p.add_argument("--launcher", type=str, default="pdsh")
    p.add_argument("--launcher_args", type=str, default="")
    p.add_argument("--force_multi", action="store_true")
    p.add_argument("--no_ssh_check", action="store_true")
    p.add_argument("--autotuning", type=str, default="")
    p.add_argument("--comment", type=str, default="")
    p.add_argument("--account", type=str, default="")
    p.add_argument("--node_rank", type=int, default=-1, help="set by the multi-node fan-out")
    p.add_argument("--world_info", type=str, default="", help="host:slots,... set by the multi-node fan-out")
    p.add_argument("--dry_run", action="store_true")
    p.add_argument("user_script", type=str)
    p.add_argument("user_args", nargs=argparse.REMAINDER)
    return p.parse_args(argv)


def fetch_hostfile(path):
    """-> OrderedDict host -> slots, or None when the file does not exist."""
    if not path or not os.path.isfile(path):
        return None
    pool = OrderedDict()
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            try:
                host, slots = line.split()
                key, n = slots.split("=")
                assert key == "slots"
                n = int(n)
            except Exception as e:  # noqa: BLE001
                raise ValueError(f"Hostfile is not formatted correctly, unable to proceed with training: {line!r}") from e
            if host in pool:
                raise ValueError(f"host {host} is already defined")
            pool[host] = n
    return pool


def _parse_filter(spec):
    out = OrderedDict()
    for node in filter(None, spec.split("@")):
        if ":" in node:
            host, devs = node.split(":")
            out[host] = [int(d) for d in devs.split(",")]
        else:
            out[node] = None
    return out


def parse_resource_filter(pool, include="", exclude=""):
    """host -> slots  =>  host -> list of device ids after ``include`` / ``exclude``."""
    if include and exclude:
        raise ValueError("include_str and exclude_str are mutually exclusive.")
    full = OrderedDict((h, list(range(n))) for h, n in pool.items())
    if include:
        inc = _parse_filter(include)
        out = OrderedDict()
        for h, devs in inc.items():
            if h not in full:
                raise ValueError(f"Hostname '{h}' not found in hostfile")
            for d in devs or []:
                if d not in full[h]:
                    raise ValueError(f"No slot '{d}' specified on host '{h}'")
            out[h] = devs if devs is not None else full[h]
        return out
    if exclude:
        exc = _parse_filter(exclude)
        for h, devs in exc.items():
            if h not in full:
                raise ValueError(f"Hostname '{h}' not found in hostfile")
            if devs is None:
                del full[h]
            else:
                for d in devs:
                    if d not in full[h]:
                        raise ValueError(f"No slot '{d}' specified on host '{h}'")
                full[h] = [d for d in full[h] if d not in devs]
                if not full[h]:
                    del full[h]
    return full


def _local_gpu_count():
    try:
        import torch
        n = torch.cuda.device_count()
        return n if n > 0 else 1
    except Exception:  # noqa: BLE001
        return 1


def run_local(script, script_args, devices, node_rank, node_sizes, master_addr, master_port, env=None):
    """Spawn one child per entry of ``devices``; returns the first non-zero exit code (0 if none)."""
    world = sum(node_sizes)
    base = sum(node_sizes[:node_rank])
    procs = []
    for local_rank, dev in enumerate(devices):
        e = dict(os.environ if env is None else env)
        e.update(RANK=str(base + local_rank), LOCAL_RANK=str(local_rank), WORLD_SIZE=str(world),
                 MASTER_ADDR=master_addr, MASTER_PORT=str(master_port), LOCAL_WORLD_SIZE=str(len(devices)),
                 NODE_RANK=str(node_rank))
        if "CUDA_VISIBLE_DEVICES" not in e and dev is not None and devices != list(range(len(devices))):
            e["NEOX_DEVICE_MAP"] = ",".join(str(d) for d in devices)
        cmd = [sys.executable, "-u", script, f"--local_rank={local_rank}"] + list(script_args)
        procs.append(subprocess.Popen(cmd, env=e))
    pidfile = os.environ.get("NEOX_PIDFILE", f"/tmp/gpt_neox_b200.{os.getuid()}.pids")
    try:                                   # read by cluster/kill.sh, which ends exactly these processes
        with open(pidfile, "w") as f:
            f.write("\n".join(str(p.pid) for p in procs) + "\n")
    except OSError:
        pidfile = None
    rc = 0
    alive = list(procs)
    try:
        while alive:
            for p in list(alive):
                r = p.poll()
                if r is None:
                    continue
                alive.remove(p)
                if r != 0 and rc == 0:
                    rc = r
                    for q in alive:           # a failed rank ends the job: stop exactly our children
                        q.send_signal(signal.SIGTERM)
            time.sleep(0.05)
    except KeyboardInterrupt:
        for q in alive:
            q.send_signal(signal.SIGTERM)
        rc = 130
    for p in procs:
        try:
            p.wait(timeout=30)
        except subprocess.TimeoutExpired:
            p.kill()
    if pidfile and os.path.exists(pidfile):
        os.remove(pidfile)
    return rc


def _exports():
    out = []
    for k, v in os.environ.items():
        if any(k.startswith(pfx) for pfx in EXPORT_ENVS) or k == "WANDB_API_KEY":
            out.append((k, v))
    return out


def build_multinode_cmd(args, active):
    """Command line(s) that start this module with ``--node_rank`` on every host of ``active``."""
    hosts = list(active)
    world_info = ",".join(f"{h}:{'.'.join(str(d) for d in devs)}" for h, devs in active.items())
    master = args.master_addr or hosts[0]
    inner = [sys.executable, "-u", "-m", "gpt_neox_b200.launcher", f"--world_info={world_info}",
             f"--master_addr={master}", f"--master_port={args.master_port}"]
    tail = [args.user_script] + list(args.user_args)
    exports = " ".join(f"export {k}={shlex.quote(v)};" for k, v in _exports())
    cwd = os.path.abspath(".")
    extra = shlex.split(args.launcher_args) if args.launcher_args else []
    name = args.launcher.lower()
    if name == "pdsh":
        remote = f"{exports} cd {shlex.quote(cwd)}; " + " ".join(shlex.quote(x) for x in inner) + \
                 " --node_rank=%n " + " ".join(shlex.quote(x) for x in tail)
        return ["pdsh", "-S", "-f", "1024", "-w", ",".join(hosts)] + extra + [remote]
    if name in ("openmpi", "mvapich"):
        cmd = ["mpirun", "-n", str(len(hosts)), "--host" if name == "openmpi" else "-hosts", ",".join(hosts)] + extra
        for k, v in _exports():
            cmd += ["-x", f"{k}={v}"] if name == "openmpi" else ["-env", k, v]
        return cmd + inner + ["--node_rank=-2"] + tail        # -2: take the node rank from the MPI environment
    if name == "slurm":
        cmd = ["srun", "-N", str(len(hosts)), "--ntasks-per-node=1", "--nodelist", ",".join(hosts)]
        if args.comment:
            cmd += ["--comment", args.comment]
        if args.account:
            cmd += ["--account", args.account]
        return cmd + extra + inner + ["--node_rank=-2"] + tail
    raise NotImplementedError(f"Unknown launcher {args.launcher}")


def _node_rank_from_env():
    for k in ("SLURM_NODEID", "OMPI_COMM_WORLD_RANK", "MV2_COMM_WORLD_RANK", "PMI_RANK"):
        if k in os.environ:
            return int(os.environ[k])
    raise RuntimeError("cannot determine the node rank from the environment")


def _job_size(args):
    """Number of processes the job would start (for the autotuner's data-parallel degree)."""
    pool = fetch_hostfile(args.hostfile)
    if not pool:
        if args.include or args.exclude:
            active = parse_resource_filter({"localhost": _local_gpu_count()}, args.include, args.exclude)
            return sum(len(d) for d in active.values())
        return args.num_gpus if args.num_gpus > 0 else _local_gpu_count()
    active = parse_resource_filter(pool, args.include, args.exclude)
    if args.num_nodes > 0:
        active = OrderedDict(list(active.items())[:args.num_nodes])
    if args.num_gpus > 0:
        active = OrderedDict((h, d[:args.num_gpus]) for h, d in active.items())
    return sum(len(d) for d in active.values())


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    args = parse_args(argv)
    if args.autotuning and not args.world_info:
        # trial runs, then (mode "run") the job itself, each through this same entry without the flag
        from . import autotuning
        if args.autotuning not in ("tune", "run"):
            raise ValueError("--autotuning takes 'tune' or 'run'")
        head = argv[:len(argv) - len(args.user_args)]
        i = head.index("--autotuning") if "--autotuning" in head else None
        if i is not None:
            del head[i:i + 2]
        else:
            head = [a for a in head if not a.startswith("--autotuning=")]
        return autotuning.run_from_launcher(args.autotuning, list(args.user_args), _job_size(args),
                                            lambda user_args: main(head + list(user_args)))
    if args.world_info:                                   # second level: we are on one host of the job
        hosts = OrderedDict()
        for item in args.world_info.split(","):
            h, devs = item.split(":")
            hosts[h] = [int(d) for d in devs.split(".")]
        rank = args.node_rank if args.node_rank >= 0 else _node_rank_from_env()
        devs = list(hosts.values())[rank]
        return run_local(args.user_script, args.user_args, devs, rank, [len(v) for v in hosts.values()],
                         args.master_addr, args.master_port)
    pool = fetch_hostfile(args.hostfile)
    if not pool:
        n = args.num_gpus if args.num_gpus > 0 else _local_gpu_count()
        if args.include or args.exclude:
            active = parse_resource_filter({"localhost": _local_gpu_count()}, args.include, args.exclude)
            devs = list(active.values())[0]
        else:
            devs = list(range(n))
        return run_local(args.user_script, args.user_args, devs, 0, [len(devs)], args.master_addr or "127.0.0.1",
                         args.master_port)
    active = parse_resource_filter(pool, args.include, args.exclude)
    if args.num_nodes > 0:
        active = OrderedDict(list(active.items())[:args.num_nodes])
    if args.num_gpus > 0:
        active = OrderedDict((h, d[:args.num_gpus]) for h, d in active.items())
    if len(active) == 1 and not args.force_multi:
        devs = list(active.values())[0]
        return run_local(args.user_script, args.user_args, devs, 0, [len(devs)], args.master_addr or "127.0.0.1",
                         args.master_port)
    cmd = build_multinode_cmd(args, active)
    if args.dry_run:
        print(" ".join(shlex.quote(c) for c in cmd))
        return 0
    return subprocess.call(cmd)


if __name__ == "__main__":
    sys.exit(main())
