"""The ``lbann`` executable of this framework: ``python -m lbann_b200.driver --prototext=...``.

Process start -> options -> communicator -> trainer -> model -> train -> test, the sequence
of src/drivers/lbann.cpp:74-233.  One process per GPU; multi-rank jobs are started with
``python -m torch.distributed.run`` (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the
environment).  On any exception a stack trace is written (optionally to
``stack_trace_rank<r>.txt``) and the whole job is aborted.
"""
from __future__ import annotations

import os
import signal
import sys
import time
import traceback
from typing import List, Optional

from google.protobuf import text_format

from .proto import lbann_pb2 as pb
from .utils import options as opts


def load_prototext(path: str):
    msg = pb.LbannPB()
    with open(path, "rb") as f:
        data = f.read()
    if path.endswith((".bin", ".protobin")):
        msg.ParseFromString(data)
    else:
        text_format.Parse(data.decode(), msg)
    return msg


def apply_overrides(msg, o: opts.Options):
    """Command-line overrides patched into the experiment (src/proto/proto_common.cpp)."""
    if o.get_int("mini_batch_size"):
        msg.trainer.mini_batch_size = o.get_int("mini_batch_size")
    if o.get_int("num_epochs") >= 0 and o.get("num_epochs") not in (None, -1):
        msg.model.num_epochs = o.get_int("num_epochs")
    if o.get_int("random_seed"):
        msg.trainer.random_seed = o.get_int("random_seed")
    if o.get_bool("disable_cuda"):
        msg.model.disable_cuda = True
    if o.get_bool("serialize_io"):
        msg.trainer.serialize_io = True
    for r in msg.data_reader.reader:
        role = {"validate": "validate", "validation": "validate"}.get(r.role, r.role)
        for key, field in (("data_filedir", "data_filedir"), (f"data_filedir_{role}", "data_filedir"),
                           (f"data_filename_{role}", "data_filename"),
                           (f"label_filename_{role}", "label_filename"),
                           (f"sample_list_{role}", "sample_list")):
            v = o.get(key)
            if v:
                setattr(r, field, v)
        if o.get("data_reader_fraction"):
            r.fraction_of_data_to_use = float(o.get("data_reader_fraction"))
        if o.get_int("absolute_sample_count"):
            r.absolute_sample_count = o.get_int("absolute_sample_count")
    ck = o.get("ckpt_dir") or o.get("checkpoint_dir")
    rs = o.get("restart_dir")
    if ck or rs:
        for cb in list(msg.trainer.callback) + list(msg.model.callback):
            if cb.HasField("checkpoint"):
                if ck:
                    cb.checkpoint.checkpoint_dir = ck
                if rs:
                    cb.checkpoint.restart_dir = rs
    return msg


def save_session(msg, argv, work_dir="."):
    """Effective prototext and command line, written once at start-up
    (src/utils/lbann_library.cpp:418-420)."""
    stamp = time.strftime("%Y%m%d_%H%M%S")
    path = os.path.join(work_dir, f"lbann_session_{stamp}.prototext")
    with open(path, "w") as f:
        f.write("# " + " ".join(argv) + "\n")
        f.write(text_format.MessageToString(msg))
    return path


def _install_signal_handlers(rank: int, to_file: bool):
    def handler(signum, frame):
        text = f"rank {rank} caught signal {signum}\n" + "".join(traceback.format_stack(frame))
        sys.stderr.write(text)
        if to_file:
            with open(f"stack_trace_rank{rank}.txt", "w") as f:
                f.write(text)
        os._exit(128 + signum)
    for s in (signal.SIGTERM, signal.SIGINT, signal.SIGABRT):
        try:
            signal.signal(s, handler)
        except (ValueError, OSError):
            pass


def run_experiment(msg, *, argv: Optional[List[str]] = None, work_dir: str = ".",
                   procs_per_trainer: int = 0, return_trainer: bool = False):
    """Train and test the experiment in this process (one rank of the job)."""
    from .exec.trainer import ExecTrainer
    o = opts.current()
    trainer = ExecTrainer(msg, procs_per_trainer=procs_per_trainer)
    comm = trainer.comm
    if not o.get_bool("disable_signal_handler"):
        _install_signal_handlers(comm.rank_in_world, o.get_bool("stack_trace_to_file"))
    try:
        model = trainer.build_model(msg.model)
        if comm.am_world_master() and o.get_bool("verbose"):
            print(model.describe(), flush=True)
        if o.get_bool("exit_after_setup"):
            return (trainer, model) if return_trainer else 0
        trainer.train(model)
        trainer.evaluate(model, "testing")
        if return_trainer:
            return trainer, model
        return 0
    except BaseException:
        text = f"rank {comm.rank_in_world}:\n" + traceback.format_exc()
        sys.stderr.write(text)
        if o.get_bool("stack_trace_to_file"):
            with open(os.path.join(work_dir, f"stack_trace_rank{comm.rank_in_world}.txt"), "w") as f:
                f.write(text)
        if comm.world_size > 1:
            os._exit(1)       # abort semantics: the launcher tears the other ranks down
        raise
    finally:
        if not return_trainer:
            trainer.shutdown()


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    o = opts.reset()
    rest = o.parse(argv)
    if "--help" in rest or "-h" in rest:
        print("usage: python -m lbann_b200.driver --prototext=<file> [options]\n" + o.describe())
        return 0
    path = o.get("prototext")
    if not path:
        parts = [o.get("model"), o.get("reader"), o.get("optimizer")]
        if not all(parts):
            print("error: --prototext (or --model, --reader and --optimizer) is required", file=sys.stderr)
            return 2
        msg = pb.LbannPB()
        for p in parts:
            msg.MergeFrom(load_prototext(p))
    else:
        rank = int(os.environ.get("RANK", "0"))
        ppt = o.get_int("procs_per_trainer")
        if o.get_bool("generate_multi_proto") and ppt > 0 and "trainer0" in path:
            # one experiment file per trainer: <prefix>trainer0<suffix> names trainer 0's and
            # trainer i reads <prefix>trainer<i><suffix> (src/proto/proto_common.cpp, used by
            # python/lbann/contrib/hyperparameter.py:80-88)
            head, _, tail = path.rpartition("trainer0")
            path = f"{head}trainer{rank // ppt}{tail}"
        msg = load_prototext(path)
    apply_overrides(msg, o)
    rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        try:
            save_session(msg, ["lbann"] + argv)
        except OSError:
            pass
    rc = run_experiment(msg, argv=argv, procs_per_trainer=o.get_int("procs_per_trainer"))
    return int(rc or 0)


if __name__ == "__main__":
    sys.exit(main())
