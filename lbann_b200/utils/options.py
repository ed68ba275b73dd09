"""Typed flags and options with ``LBANN_<NAME>`` environment fallbacks.

Resolution order, later wins: built-in default < environment (``LBANN_`` + upper-cased
name) < command line / explicit ``set``.  The option names are the reference's
(include/lbann/utils/options.hpp, src/utils/options.cpp:33-573); a few extra knobs of this
framework (default dtype, CUDA graph capture) follow the same scheme.
"""
from __future__ import annotations

import argparse
import os
from typing import Any, Dict, List, Optional

_FLAGS = [
    "disable_cuda", "disable_distconv", "disable_signal_handler", "exit_after_setup",
    "generate_multi_proto", "ltfb", "ltfb_verbose", "multitrainer_verbose", "preload_data_store",
    "print_affinity", "serialize_io", "stack_trace_to_file", "disable_cudnn_tensor_ops",
    "use_data_store", "verbose", "no_inplace", "no_backprop_disable", "random_init_models_identically",
    "data_store_cache", "data_store_debug", "data_store_fail", "data_store_profile",
    "check_data", "keep_sample_order", "quiet", "write_sample_list", "z_score", "use_cuda_graph",
    "allow_multitrainer_global_statistics", "hang", "use_caliper", "deterministic",
    "trainer_enable_subgrid_async_comm",       # K-FAC: factor inversions run beside the next step
    # accepted for command lines written for the reference; what they switch (its data-store
    # test modes, SHMEM / NVSHMEM start-up, GPU-direct forward prop, the second model of its
    # sub-grid scheme) has no counterpart here
    "disable_background_io_activity", "ltfb_allow_global_statistics", "ltfb_global_multitrainer_statistics",
    "use_gpu_direct_memory_in_forward_prop", "init_shmem", "init_nvshmem", "caliper",
    "data_store_min_max_timing", "data_store_no_thread", "data_store_test_cache", "node_sizes_vary",
    "keep_packed_fields", "load_full_sample_list_once", "write_sample_label_list", "jag",
    "trainer_create_two_models", "trainer_enable_topo_aware_subgrid",
]
_OPTIONS = {
    # name: (type, default)
    "ckpt_dir": (str, ""), "restart_dir": (str, ""), "load_model_weights_dir": (str, ""),
    "data_store_spill": (str, ""),      # directory: stores load their spilled cache from it and write it back at the end
    "load_model_weights_dir_is_complete": (int, 0), "hydrogen_block_size": (int, 0),
    "metadata": (str, ""), "mini_batch_size": (int, 0), "model": (str, ""), "num_epochs": (int, -1),
    "num_io_threads": (int, 0), "max_rng_seeds": (int, 0), "optimizer": (str, ""),
    "procs_per_trainer": (int, 0), "prototext": (str, ""), "random_seed": (int, 0),
    "reader": (str, ""), "trainer_grid_height": (int, 0), "trainer_primary_grid_size": (int, 0),
    "num_subgrids": (int, 0), "num_subgrids_block_order": (int, 0), "caliper_config": (str, ""),
    "absolute_sample_count": (int, 0), "data_filedir": (str, ""), "data_filedir_test": (str, ""),
    "data_filedir_train": (str, ""), "data_filedir_validate": (str, ""),
    "data_filename_test": (str, ""), "data_filename_train": (str, ""),
    "data_filename_validate": (str, ""), "data_reader_fraction": (float, 0.0),
    "label_filename_test": (str, ""), "label_filename_train": (str, ""),
    "label_filename_validate": (str, ""), "sample_list_test": (str, ""),
    "sample_list_train": (str, ""), "sample_list_validate": (str, ""),
    "sequence_length": (int, 0), "vocab": (str, ""), "default_dtype": (str, ""),
    "num_train_samples": (int, 0), "num_validate_samples": (int, 0), "num_test_samples": (int, 0),
    "checkpoint_dir": (str, ""), "rng_seeds_per_trainer_to_display": (int, 2), "max_io_thread_rngs": (int, 128),
    "omp_num_threads": (int, 4), "data_store_test_checkpoint": (str, ""), "normalization": (str, ""),
    "pilot2_read_file_sizes": (str, ""), "pilot2_save_file_sizes": (str, ""),
    "smiles_buffer_size": (int, 16 * 1024 * 1024),
    # options of the reference's data-preparation tools that share its parser
    "base_dir": (str, ""), "filelist": (str, ""), "filename": (str, ""), "format": (str, ""),
    "index_fn": (str, ""), "mapping_fn": (str, ""), "num_lists": (int, -1), "num_samples": (int, -1),
    "num_samples_per_file": (int, 1000), "num_samples_per_list": (int, -1), "num_subdirs": (int, -1),
    "output_base_dir": (str, ""), "output_base_fn": (str, ""), "output_dir": (str, ""), "output_fn": (str, ""),
    "samples_per_file": (int, -1),
}


class Options:
    def __init__(self):
        self._values: Dict[str, Any] = {}

    @staticmethod
    def _env(name: str) -> Optional[str]:
        return os.environ.get("LBANN_" + name.upper())

    def set(self, name: str, value: Any):
        self._values[name] = value

    def get(self, name: str, default: Any = None) -> Any:
        if name in self._values:
            return self._values[name]
        env = self._env(name)
        if env is not None:
            if name in _OPTIONS:
                return _OPTIONS[name][0](env)
            return env
        if name in _OPTIONS:
            return _OPTIONS[name][1]
        return default

    def get_bool(self, name: str) -> bool:
        if name in self._values:
            return bool(self._values[name])
        env = self._env(name)
        if env is not None:
            return env.strip().lower() not in ("", "0", "false", "no", "off")
        return False

    def get_int(self, name: str) -> int:
        v = self.get(name, 0)
        try:
            return int(v)
        except (TypeError, ValueError):
            return 0

    def parse(self, argv: List[str]) -> List[str]:
        """Parse known ``--flag`` / ``--option=value`` arguments; returns the rest."""
        ap = argparse.ArgumentParser(add_help=False, allow_abbrev=False)
        for f in _FLAGS:
            ap.add_argument(f"--{f}", action="store_true", default=None)
        for n, (tp, _) in _OPTIONS.items():
            ap.add_argument(f"--{n}", type=tp, default=None)
        ns, rest = ap.parse_known_args(argv)
        for k, v in vars(ns).items():
            if v is not None:
                self._values[k] = v
        return rest

    def describe(self) -> str:
        lines = ["Flags:"] + [f"  --{f}  [env LBANN_{f.upper()}]" for f in _FLAGS]
        lines += ["Options:"] + [f"  --{n}=<{tp.__name__}> (default {d!r})  [env LBANN_{n.upper()}]"
                                 for n, (tp, d) in _OPTIONS.items()]
        return "\n".join(lines)


_current = Options()


def current() -> Options:
    return _current


def reset():
    global _current
    _current = Options()
    return _current
