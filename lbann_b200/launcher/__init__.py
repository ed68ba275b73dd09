"""``lbann.run`` and batch-script generation.

``run`` writes the experiment prototext into a work directory and executes it.  The default
launcher runs the experiment on this node: in-process for one rank, through
``python -m torch.distributed.run`` (one process per GPU) for several.  Scheduler back ends
(slurm, lsf, flux, pjm, openmpi) generate and optionally submit a batch script that starts
the same driver under the site's parallel launcher, as the reference's launcher package
does (python/lbann/launcher/__init__.py:52-197, batch_script.py, slurm.py, lsf.py, flux.py,
pjm.py, openmpi.py).
"""
from __future__ import annotations

import datetime
import os
import shutil
import subprocess
import sys
from typing import Dict, List, Optional

from ..proto.serialize import save_prototext
from .batch_script import (BatchScript, FluxBatchScript, LSFBatchScript, OpenMPIBatchScript,
                           PJMBatchScript, SlurmBatchScript, TorchrunBatchScript, make_batch_script)

__all__ = ["run", "make_batch_script", "make_timestamped_work_dir", "BatchScript",
           "SlurmBatchScript", "LSFBatchScript", "FluxBatchScript", "PJMBatchScript",
           "OpenMPIBatchScript", "TorchrunBatchScript"]


def make_timestamped_work_dir(work_dir=None, job_name="lbann", base=None):
    if work_dir:
        os.makedirs(work_dir, exist_ok=True)
        return os.path.realpath(work_dir)
    base = base or os.environ.get("LBANN_EXPERIMENT_DIR") or os.getcwd()
    stamp = datetime.datetime.now().strftime("%Y%m%d_%H%M%S")
    path = os.path.join(base, f"{stamp}_{job_name}")
    i = 1
    cand = path
    while os.path.exists(cand):
        cand = f"{path}_{i}"
        i += 1
    os.makedirs(cand)
    return os.path.realpath(cand)


def detect_scheduler() -> str:
    if "SLURM_JOB_ID" in os.environ or shutil.which("srun"):
        return "slurm"
    if "LSB_JOBID" in os.environ or shutil.which("jsrun"):
        return "lsf"
    if "FLUX_URI" in os.environ:
        return "flux"
    if shutil.which("pjsub"):
        return "pjm"
    return "local"


def run(trainer, model, data_reader, optimizer, work_dir=None, proto_file_name=None, nodes=1,
        procs_per_node=1, time_limit=None, scheduler=None, job_name="lbann", partition=None,
        account=None, reservation=None, launcher=None, launcher_args=(), lbann_exe=None,
        lbann_args=(), procs_per_trainer=None, environment=None, overwrite_script=False,
        setup_only=False, batch_job=False, nvprof=False, nvprof_output_name=None,
        binary_protobuf=False, experiment_dir=None):
    """Run an experiment; returns the exit status (0 = success)."""
    work_dir = make_timestamped_work_dir(experiment_dir or work_dir, job_name)
    proto_file_name = proto_file_name or ("experiment.protobin" if binary_protobuf
                                          else "experiment.prototext")
    proto_file = os.path.join(work_dir, proto_file_name)
    save_prototext(proto_file, binary=binary_protobuf, trainer=trainer, model=model,
                   data_reader=data_reader, optimizer=optimizer)
    lbann_args = list(lbann_args) if not isinstance(lbann_args, str) else lbann_args.split()
    args = [f"--prototext={proto_file}"] + lbann_args
    if procs_per_trainer:
        args.append(f"--procs_per_trainer={procs_per_trainer}")
    scheduler = scheduler or detect_scheduler()
    nprocs = nodes * procs_per_node
    env = dict(environment or {})

    if scheduler == "local" and nprocs == 1 and not batch_job and launcher is None:
        if setup_only:
            return 0
        old_env = {k: os.environ.get(k) for k in env}
        os.environ.update({k: str(v) for k, v in env.items()})
        cwd = os.getcwd()
        os.chdir(work_dir)
        try:
            from .. import driver
            return driver.main(args)
        finally:
            os.chdir(cwd)
            for k, v in old_env.items():
                if v is None:
                    os.environ.pop(k, None)
                else:
                    os.environ[k] = v

    script = make_batch_script(work_dir=work_dir, nodes=nodes, procs_per_node=procs_per_node,
                               time_limit=time_limit, scheduler=scheduler, job_name=job_name,
                               partition=partition, account=account, reservation=reservation,
                               launcher=launcher, launcher_args=list(launcher_args),
                               environment=env)
    exe = [lbann_exe] if lbann_exe else [sys.executable, "-m", "lbann_b200.driver"]
    cmd = exe + args
    if nvprof:
        out = nvprof_output_name or os.path.join(work_dir, "nvprof_output.%q{RANK}.nvvp")
        cmd = ["nsys", "profile", "-o", out] + cmd
    script.add_parallel_command(cmd)
    script.write(overwrite=overwrite_script)
    if setup_only:
        return 0
    return script.submit() if batch_job else script.run()
