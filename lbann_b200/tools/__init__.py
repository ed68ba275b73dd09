"""Stand-alone data-preparation utilities (the reference's ``tools/`` directory):

* ``python -m lbann_b200.tools.partition_input_list``  shuffle a "path label" list and cut
  it into equal partitions (tools/partition_input_list.cpp);
* ``python -m lbann_b200.tools.compute_mean``  per-pixel mean image / per-channel mean of an
  image list, optionally after a centre crop, computed by several ranks
  (tools/compute_mean/compute_mean.cpp, uniform_mean.cpp);
* ``python -m lbann_b200.tools.mnist_to_npy``  MNIST idx files to ``.npy`` / ``.npz``
  (tools/mnist/mnist_to_npy_and_npz.py).
"""
