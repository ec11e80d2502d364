#!/usr/bin/env python
"""Image classification with compressed gradient all-reduce (CIFAR-shaped data).

Counterpart of the reference's ``examples/ImageClassification/main.py``: same flags
(``--model``, ``--grad_reducer``, ``--start_compression_iter``, ``--compression_ratio``, ``--beta``,
``--sketch_size``, ``--matrix_approximation_rank``, ``--min_compression_rate`` ...), SGD with
Nesterov momentum, three learning-rate decay milestones, accuracy per epoch, results pickled.
Launch with ``torchrun --nproc-per-node N examples/image_classification/main.py ...`` (or as a
single process).  Without ``--data_path`` the data is synthetic: there is no dataset on the box.
"""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import conef_b200 as cb  # noqa: E402
from conef_b200 import models  # noqa: E402
from conef_b200.data import SyntheticImages  # noqa: E402
from conef_b200.utils import GracefulStop, JsonLogger, make_directory, save_obj  # noqa: E402

MODELS = {
    "resnet20": models.ResNet20, "resnet18": models.ResNet18, "resnet34": models.ResNet34, "resnet50": models.ResNet50,
    "resnet101": models.ResNet101, "resnet152": models.ResNet152, "vgg16": lambda c: models.VGG("VGG16", c),
    "vgg19": lambda c: models.VGG("VGG19", c), "densenet121": models.DenseNet121, "densenet_cifar": models.densenet_cifar,
    "mobilenetv2": models.MobileNetV2, "resnext29_2x64d": models.ResNeXt29_2x64d,
    "shufflenetv2": lambda c: models.ShuffleNetV2(1, c), "lenet": models.LeNet,
    "wideresnet28_10": lambda c: models.WideResNet(28, 10, 0.3, c), "wideresnet16_4": lambda c: models.WideResNet(16, 4, 0.3, c),
}


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--model", default="resnet20", choices=sorted(MODELS))
    p.add_argument("--dataset", default="cifar10", choices=["cifar10", "cifar100"])
    p.add_argument("--data_path", default=None, help="torchvision CIFAR root; synthetic data when omitted")
    p.add_argument("--epochs", type=int, default=1)
    p.add_argument("--steps_per_epoch", type=int, default=50, help="synthetic data only")
    p.add_argument("--batch_size", type=int, default=128, help="per process")
    p.add_argument("--lr", type=float, default=0.1)
    p.add_argument("--momentum", type=float, default=0.9)
    p.add_argument("--weight_decay", type=float, default=5e-4)
    p.add_argument("--nesterov", action="store_true", default=True)
    p.add_argument("--lr_decay", type=float, default=0.1)
    p.add_argument("--grad_reducer", default="conef_powersgd", choices=cb.REDUCERS)
    p.add_argument("--start_compression_iter", type=int, default=10)
    p.add_argument("--compression_ratio", type=float, default=0.1)
    p.add_argument("--beta", type=float, default=0.9)
    p.add_argument("--sketch_size", type=float, default=0.2)
    p.add_argument("--matrix_approximation_rank", type=int, default=4)
    p.add_argument("--min_compression_rate", type=float, default=2)
    p.add_argument("--orthogonalization_epsilon", type=float, default=0)
    p.add_argument("--error_compressor", default=None)
    p.add_argument("--bf16", action="store_true")
    p.add_argument("--results", default="results/image_classification")
    p.add_argument("--seed", type=int, default=0)
    return p.parse_args()


def main():
    args = parse()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29501")
    cuda = torch.cuda.is_available()
    device = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(device)
    dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    torch.manual_seed(args.seed)
    classes = 10 if args.dataset == "cifar10" else 100
    if args.data_path:
        import torchvision
        import torchvision.transforms as T
        tf = T.Compose([T.RandomCrop(32, padding=4), T.RandomHorizontalFlip(), T.ToTensor()])
        ds = getattr(torchvision.datasets, args.dataset.upper())(args.data_path, train=True, transform=tf)
    else:
        ds = SyntheticImages(args.steps_per_epoch * args.batch_size * world, classes)
    sampler = DistributedSampler(ds, world, rank, shuffle=True, seed=args.seed)
    loader = DataLoader(ds, args.batch_size, sampler=sampler, num_workers=2, pin_memory=cuda, drop_last=True)
    trainer = cb.DataParallelTrainer(
        MODELS[args.model](classes),
        lambda p: torch.optim.SGD(p, lr=args.lr, momentum=args.momentum, weight_decay=args.weight_decay,
                                  nesterov=args.nesterov),
        F.cross_entropy, reducer=args, device=device, autocast_dtype=torch.bfloat16 if (args.bf16 and cuda) else None,
        channels_last=cuda)
    milestones = [int(args.epochs * f) for f in (0.5, 0.75, 0.9)]
    sched = torch.optim.lr_scheduler.MultiStepLR(trainer.optimizer, milestones, args.lr_decay)
    stop, log = GracefulStop(), JsonLogger(stdout=True)
    history = []
    for epoch in range(args.epochs):
        sampler.set_epoch(epoch)
        t0, seen, correct, loss_sum = time.time(), 0, 0, 0.0
        for x, y in loader:
            loss = trainer.step(x, y)
            loss_sum += float(loss)
            seen += y.numel()
            if stop.requested:
                break
        sched.step()
        dt = time.time() - t0
        rec = dict(epoch=epoch, loss=loss_sum / max(1, len(loader)), img_per_s=seen * world / dt,
                   ef_buffer_mb=(trainer.state.ef_buffer_bytes() / 1e6) if trainer.state else 0.0)
        history.append(rec)
        log.log(epoch, **rec)
        if stop.requested:
            break
    trainer.check()
    if rank == 0:
        make_directory(args.results)
        save_obj({"args": vars(args), "history": history}, os.path.join(args.results, "results"))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
