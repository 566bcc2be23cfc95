"""The reference's training driver (StreamBrain ``train.py:44-202``) on the B200 backend.

    python -m streambrain_b200.train <mnist|fashion_mnist|stl-10> <single|double> <batch size> [data directory]

Reads the dataset files the reference reads (``train-images-idx3-ubyte`` ... for the IDX datasets,
``unlabeled_X.bin`` / ``train_X.bin`` / ``train_y.bin`` / ``test_X.bin`` / ``test_y.bin`` for STL-10) from the
data directory (default: the working directory), builds the two-layer network with the dataset's
hyper-parameters and trains / evaluates it.  Under ``torchrun`` the ranks train data-parallel (row-sharded).
"""
from __future__ import annotations

import os
import sys
import time

import numpy as np


def main(argv):
    if len(argv) not in (4, 5):
        print("Usage: python -m streambrain_b200.train <mnist/fashion_mnist/stl-10> <single/double> <batch size> [dir]")
        return 1
    dataset, precision = argv[1], (np.float32 if argv[2] == "single" else np.float64)
    batch_size = int(argv[3])
    root = argv[4] if len(argv) == 5 else "."
    import streambrain_b200 as backend
    from streambrain_b200 import datasets, hyperparameters, parallel

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    np.random.seed(0)
    path = lambda name: os.path.join(root, name)
    if dataset in ("mnist", "fashion_mnist"):
        l1_x, l1_y = datasets.load_mnist(path("train-images-idx3-ubyte"), path("train-labels-idx1-ubyte"), precision)
        l2_x, l2_y = l1_x, l1_y
        test_x, test_y = datasets.load_mnist(path("t10k-images-idx3-ubyte"), path("t10k-labels-idx1-ubyte"), precision)
    elif dataset == "stl-10":
        l1_x = datasets.load_stl_10_images(path("unlabeled_X.bin"), precision)[:15000, :]
        l1_y = np.zeros([l1_x.shape[0], 10], dtype=precision)
        l2_x, l2_y = datasets.load_stl_10_images(path("train_X.bin"), precision), datasets.load_stl_10_labels(path("train_y.bin"), precision)
        test_x, test_y = datasets.load_stl_10_images(path("test_X.bin"), precision), datasets.load_stl_10_labels(path("test_y.bin"), precision)
    else:
        print("Unknown dataset")
        return 1
    hp = hyperparameters.for_dataset(dataset, batch_size, n_inputs=l1_x.shape[1])
    if rank == 0:
        print('Dataset:', dataset, 'Batch size:', batch_size, 'precision:', precision)
    net = hyperparameters.build_network(backend, hp, precision)
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl")

        def sum_counts(a):
            t = torch.from_numpy(np.asarray(a).copy()).cuda()
            dist.all_reduce(t)
            return t.cpu().numpy()
        net.set_data_parallel(rank, world, all_reduce=lambda t: dist.all_reduce(t, async_op=True),
                              sum_counts=sum_counts, all_gather_bytes=parallel.all_gather_bytes_over(dist))
    t0 = time.time()
    net.fit(l1_x, l1_y, batch_size, [(0, hp["l1_epochs"])])
    net.fit(l2_x, l2_y, batch_size, [(1, hp["l2_epochs"])])
    t1 = time.time()
    correct, total = net.evaluate(test_x, test_y, batch_size)
    t2 = time.time()
    if rank == 0:
        print('Training duration: ' + str(t1 - t0))
        print('Testing duration:  ' + str(t2 - t1))
        print('Accuracy:          ' + str(correct / total))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
