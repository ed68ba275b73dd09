"""Exhaustive grid search over hyper-parameters, one model per trainer.

Every point of the Cartesian product of the given value lists becomes one experiment file
``run<r>.trainer<t>`` in the batch script's work directory; each run of the driver trains
``num_trainers`` of them side by side (``--generate_multi_proto``), and the table of
configurations goes to ``hyperparameters.csv``.  Same contract as the reference's helper
(python/lbann/contrib/hyperparameter.py:9-124).
"""
from __future__ import annotations

import csv
import itertools
import os
import shutil
import sys

from ..proto.serialize import save_prototext


def grid_search(script, make_experiment, procs_per_trainer=1, hyperparameters_file=None,
                run=True, **kwargs):
    """``script``: a launcher batch script (its nodes x procs_per_node ranks are divided into
    trainers of ``procs_per_trainer``).  ``make_experiment(**point)`` returns
    ``(model, optimizer, data_reader, trainer)``.  Keyword arguments: lists of values.
    Returns the rows written to the CSV file."""
    work_dir, ppn = script.work_dir, script.procs_per_node
    if ppn % procs_per_trainer and procs_per_trainer % ppn:
        raise RuntimeError(f"trainer size ({procs_per_trainer}) and ranks per node ({ppn}) "
                           "are not multiples of each other")
    num_trainers = max(script.nodes * ppn // procs_per_trainer, 1)
    keys = list(kwargs)
    points = list(itertools.product(*[kwargs[k] for k in keys]))
    rows = [["run_id", "trainer_id", "model_name"] + keys]
    os.makedirs(work_dir, exist_ok=True)
    exe = [sys.executable, "-m", "lbann_b200.driver"]

    def launch(run_id):
        script.add_parallel_command(exe + [f"--procs_per_trainer={procs_per_trainer}",
                                           "--generate_multi_proto",
                                           f"--prototext={work_dir}/run{run_id}.trainer0"])

    for model_id, values in enumerate(points):
        run_id, trainer_id = divmod(model_id, num_trainers)
        model, optimizer, reader, trainer = make_experiment(**dict(zip(keys, values)))
        if not model.name:
            model.name = f"model{model_id}"
        rows.append([run_id, trainer_id, model.name] + list(values))
        save_prototext(os.path.join(work_dir, f"run{run_id}.trainer{trainer_id}"), model=model,
                       optimizer=optimizer, data_reader=reader, trainer=trainer)
        if trainer_id == num_trainers - 1:
            launch(run_id)
    if points and trainer_id != num_trainers - 1:
        # the last run is short of trainers: repeat its last configuration so that every
        # trainer of the job has a file to read
        last = os.path.join(work_dir, f"run{run_id}.trainer{trainer_id}")
        for t in range(trainer_id + 1, num_trainers):
            shutil.copyfile(last, os.path.join(work_dir, f"run{run_id}.trainer{t}"))
            rows.append([run_id, t] + rows[-1][2:])
        launch(run_id)
    path = hyperparameters_file or os.path.join(work_dir, "hyperparameters.csv")
    with open(path, "w", newline="") as f:
        csv.writer(f).writerows(rows)
    if run:
        script.run(True)
    return rows
