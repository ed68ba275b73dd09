"""Batch scripts for the supported job launchers.

A batch script is a shell script with a scheduler header, environment exports and one or
more commands, some of them started under the parallel launcher (``srun``, ``jsrun``,
``flux run``, ``mpiexec``, ``mpirun`` or, on a single node without a scheduler,
``python -m torch.distributed.run``).  Mirrors python/lbann/launcher/{batch_script,slurm,
lsf,flux,pjm,openmpi}.py of the reference.
"""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
from typing import Dict, List, Optional


class BatchScript:
    header_prefix = "#"

    def __init__(self, script_file=None, work_dir=None, nodes=1, procs_per_node=1, time_limit=None,
                 job_name="lbann", partition=None, account=None, reservation=None, launcher=None,
                 launcher_args=None, environment=None, interpreter="/bin/bash"):
        self.work_dir = os.path.realpath(work_dir or os.getcwd())
        self.script_file = script_file or os.path.join(self.work_dir, "batch.sh")
        self.nodes, self.procs_per_node = nodes, procs_per_node
        self.time_limit = time_limit
        self.job_name, self.partition = job_name, partition
        self.account, self.reservation = account, reservation
        self.launcher = launcher
        self.launcher_args = list(launcher_args or [])
        self.out_log = os.path.join(self.work_dir, "out.log")
        self.err_log = os.path.join(self.work_dir, "err.log")
        self.header: List[str] = [f"#!{interpreter}"]
        self.body: List[str] = []
        self.add_header()
        for k, v in (environment or {}).items():
            self.add_body_line(f"export {k}={shlex.quote(str(v))}")
        self.add_body_line(f"cd {shlex.quote(self.work_dir)}")

    # -- to specialise
    def add_header(self):
        pass

    def parallel_prefix(self) -> List[str]:
        return []

    def submit_command(self) -> Optional[List[str]]:
        return None

    # -- common
    def add_header_line(self, line):
        self.header.append(line)

    def add_body_line(self, line):
        self.body.append(line)

    def add_command(self, command):
        self.add_body_line(command if isinstance(command, str) else
                           " ".join(shlex.quote(str(c)) for c in command))

    def add_parallel_command(self, command):
        cmd = command.split() if isinstance(command, str) else list(command)
        self.add_command(self.parallel_prefix() + cmd)

    def write(self, overwrite=False):
        if os.path.exists(self.script_file) and not overwrite:
            raise RuntimeError(f"batch script {self.script_file} already exists")
        os.makedirs(os.path.dirname(self.script_file), exist_ok=True)
        with open(self.script_file, "w") as f:
            f.write("\n".join(self.header) + "\n\n" + "\n".join(self.body) + "\n")
        os.chmod(self.script_file, 0o755)

    def run(self, overwrite=True) -> int:
        if not os.path.exists(self.script_file):
            self.write(overwrite)
        with open(self.out_log, "w") as out, open(self.err_log, "w") as err:
            p = subprocess.Popen(["/bin/bash", self.script_file], stdout=subprocess.PIPE,
                                 stderr=subprocess.PIPE, text=True, cwd=self.work_dir)
            so, se = p.communicate()
            out.write(so)
            err.write(se)
            sys.stdout.write(so)
            sys.stderr.write(se)
        return p.returncode

    def submit(self, overwrite=True) -> int:
        cmd = self.submit_command()
        if cmd is None:
            return self.run(overwrite)
        if not os.path.exists(self.script_file):
            self.write(overwrite)
        return subprocess.call(cmd + [self.script_file], cwd=self.work_dir)


def _hms(minutes):
    m = int(round(minutes))
    return f"{m // 60:02d}:{m % 60:02d}:00"


class SlurmBatchScript(BatchScript):
    def add_header(self):
        h = self.add_header_line
        h(f"#SBATCH --chdir={self.work_dir}")
        h(f"#SBATCH --output={self.out_log}")
        h(f"#SBATCH --error={self.err_log}")
        h(f"#SBATCH --nodes={self.nodes}")
        h(f"#SBATCH --ntasks={self.nodes * self.procs_per_node}")
        h(f"#SBATCH --ntasks-per-node={self.procs_per_node}")
        if self.time_limit is not None:
            h(f"#SBATCH --time={_hms(self.time_limit)}")
        if self.job_name:
            h(f"#SBATCH --job-name={self.job_name}")
        if self.partition:
            h(f"#SBATCH --partition={self.partition}")
        if self.account:
            h(f"#SBATCH --account={self.account}")
        if self.reservation:
            h(f"#SBATCH --reservation={self.reservation}")

    def parallel_prefix(self):
        return [self.launcher or "srun"] + self.launcher_args + [
            f"--nodes={self.nodes}", f"--ntasks={self.nodes * self.procs_per_node}",
            f"--ntasks-per-node={self.procs_per_node}"]

    def submit_command(self):
        return ["sbatch"]


class LSFBatchScript(BatchScript):
    def add_header(self):
        h = self.add_header_line
        h(f"#BSUB -cwd {self.work_dir}")
        h(f"#BSUB -o {self.out_log}")
        h(f"#BSUB -e {self.err_log}")
        h(f"#BSUB -nnodes {self.nodes}")
        if self.time_limit is not None:
            h(f"#BSUB -W {int(round(self.time_limit))}")
        if self.job_name:
            h(f"#BSUB -J {self.job_name}")
        if self.partition:
            h(f"#BSUB -q {self.partition}")
        if self.account:
            h(f"#BSUB -G {self.account}")
        if self.reservation:
            h(f"#BSUB -U {self.reservation}")

    def parallel_prefix(self):
        return [self.launcher or "jsrun"] + self.launcher_args + [
            "--nrs", str(self.nodes), "--rs_per_host", "1", "--tasks_per_rs",
            str(self.procs_per_node), "--gpu_per_rs", "ALL_GPUS", "--cpu_per_rs", "ALL_CPUS"]

    def submit_command(self):
        return ["bsub"]


class FluxBatchScript(BatchScript):
    def add_header(self):
        h = self.add_header_line
        h(f"#flux: --nodes={self.nodes}")
        h(f"#flux: --output={self.out_log}")
        h(f"#flux: --error={self.err_log}")
        if self.time_limit is not None:
            h(f"#flux: --time-limit={int(round(self.time_limit))}m")
        if self.job_name:
            h(f"#flux: --job-name={self.job_name}")
        if self.partition:
            h(f"#flux: --queue={self.partition}")

    def parallel_prefix(self):
        return [self.launcher or "flux", "run"] + self.launcher_args + [
            f"-N{self.nodes}", f"-n{self.nodes * self.procs_per_node}", "--exclusive"]

    def submit_command(self):
        return ["flux", "batch"]


class PJMBatchScript(BatchScript):
    def add_header(self):
        h = self.add_header_line
        h(f'#PJM -L "node={self.nodes}"')
        h(f'#PJM --mpi "max-proc-per-node={self.procs_per_node}"')
        h(f"#PJM -o {self.out_log}")
        h(f"#PJM -e {self.err_log}")
        if self.time_limit is not None:
            h(f'#PJM -L "elapse={_hms(self.time_limit)}"')
        if self.job_name:
            h(f"#PJM -N {self.job_name}")
        if self.partition:
            h(f'#PJM -L "rscgrp={self.partition}"')
        if self.account:
            h(f"#PJM -g {self.account}")

    def parallel_prefix(self):
        return [self.launcher or "mpiexec"] + self.launcher_args + [
            "-n", str(self.nodes * self.procs_per_node)]

    def submit_command(self):
        return ["pjsub"]


class OpenMPIBatchScript(BatchScript):
    def parallel_prefix(self):
        return [self.launcher or "mpirun"] + self.launcher_args + [
            "-n", str(self.nodes * self.procs_per_node), "--map-by",
            f"ppr:{self.procs_per_node}:node"]


class TorchrunBatchScript(BatchScript):
    """Single-node launcher of this framework: one process per GPU over NCCL / gloo."""

    def parallel_prefix(self):
        port = 29500 + (os.getpid() % 2000)
        return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                f"--nproc-per-node={self.procs_per_node}", "--master-addr", "127.0.0.1",
                "--master-port", str(port)] + self.launcher_args

    def add_parallel_command(self, command):
        cmd = command.split() if isinstance(command, str) else list(command)
        # torchrun starts a script or module itself: drop a leading interpreter
        if cmd and os.path.basename(cmd[0]).startswith("python"):
            cmd = cmd[1:]
        self.add_command(self.parallel_prefix() + cmd)


_SCRIPTS = {"slurm": SlurmBatchScript, "lsf": LSFBatchScript, "flux": FluxBatchScript,
            "pjm": PJMBatchScript, "openmpi": OpenMPIBatchScript, "local": TorchrunBatchScript,
            "torchrun": TorchrunBatchScript}


def make_batch_script(scheduler="local", **kwargs) -> BatchScript:
    key = (scheduler or "local").lower()
    if key not in _SCRIPTS:
        raise RuntimeError(f"unsupported job scheduler ({scheduler})")
    return _SCRIPTS[key](**kwargs)
