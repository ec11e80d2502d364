#!/usr/bin/env python
"""Image classification with compressed gradient all-reduce (CIFAR-shaped data).

Counterpart of the reference's ``examples/ImageClassification/main.py``: same flags
(``--model``, ``--grad_reducer``, ``--start_compression_iter``, ``--compression_ratio``, ``--beta``,
``--sketch_size``, ``--matrix_approximation_rank``, ``--min_compression_rate`` ...), SGD with
Nesterov momentum, three learning-rate decay epochs, test accuracy after every epoch on rank 0
(``main.py:238-257,300-306``), and the results folder the reference writes (``main.py:23-66``):
``train_losses.pkl``, ``test_accuracies.pkl``, ``time_per_epoch.pkl`` and a ``README.md`` listing the
run's settings and best accuracy, appended to instead of overwritten with ``--resume``.
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
from conef_b200.optim import FusedSGD  # noqa: E402
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
    p.add_argument("--lr_decay_ratio", type=float, default=10, help="the learning rate is divided by this ...")
    p.add_argument("--lr_decay_at_epoch1", type=int, default=None, help="... at these epochs (default: 53 %%, 80 %%")
    p.add_argument("--lr_decay_at_epoch2", type=int, default=None, help="and 100 %% of --epochs, the reference's")
    p.add_argument("--lr_decay_at_epoch3", type=int, default=None, help="80 / 120 / 150 of 150)")
    p.add_argument("--test_steps", type=int, default=10, help="synthetic data only: test batches per epoch")
    p.add_argument("--name", default="image_classification", help="results go to <results>/<name>")
    p.add_argument("-r", "--resume", type=int, default=0, help="1: append to the results README of an earlier run")
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
    p.add_argument("--cuda_graphs", action="store_true",
                   help="replay the forward and backward passes of the model's blocks as CUDA graphs (fixed batch size)")
    p.add_argument("--no_cudnn_autotune", action="store_true",
                   help="keep cuDNN's heuristic choice of convolution engines instead of timing them on first use")
    p.add_argument("--results", default="results")
    p.add_argument("--seed", type=int, default=0)
    return p.parse_args()


def evaluate(net, loader, device, autocast_dtype=None, channels_last=False) -> float:
    """Top-1 accuracy in percent over ``loader`` (the reference's ``test``, main.py:238-257)."""
    was_training = net.training
    net.eval()
    correct = total = 0
    with torch.no_grad():
        for x, y in loader:
            x, y = x.to(device, non_blocking=True), y.to(device, non_blocking=True)
            if channels_last:
                x = x.contiguous(memory_format=torch.channels_last)
            with torch.autocast(device.type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
                out = net(x)
            correct += int(out.argmax(1).eq(y).sum())
            total += y.numel()
    net.train(was_training)
    return 100.0 * correct / max(1, total)


def write_results(args, result, world) -> str:
    """The reference's results folder (main.py:23-66): three pickles and a README of the settings."""
    directory = os.path.join(args.results, args.name)
    make_directory(directory)
    save_obj(result["train_losses"], os.path.join(directory, "train_losses"))
    save_obj(result["test_accuracies"], os.path.join(directory, "test_accuracies"))
    save_obj(result["time"], os.path.join(directory, "time_per_epoch"))
    save_obj({"args": vars(args), "history": result["history"]}, os.path.join(directory, "results"))
    summary = dict(model=args.model, dataset=args.dataset, opt="SGD", lr=args.lr, batch_size=args.batch_size,
                   world_size=world, momentum=args.momentum, nesterov=args.nesterov, weight_decay=args.weight_decay,
                   grad_reducer=args.grad_reducer, matrix_approximation_rank=args.matrix_approximation_rank,
                   beta=args.beta, sketch_size=args.sketch_size,
                   best_acc=max(result["test_accuracies"]) if result["test_accuracies"] else 0)
    with open(os.path.join(directory, "README.md"), "a" if args.resume else "w") as f:
        if args.resume:
            f.write("\n")
        for key, val in summary.items():
            f.write(f"{key}: {val}\\\n")
    return directory


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
        test_ds = getattr(torchvision.datasets, args.dataset.upper())(args.data_path, train=False, transform=T.ToTensor())
    else:
        ds = SyntheticImages(args.steps_per_epoch * args.batch_size * world, classes)
        test_ds = SyntheticImages(args.test_steps * args.batch_size, classes, seed=args.seed + 7919)
    test_loader = DataLoader(test_ds, args.batch_size, shuffle=False, num_workers=2, pin_memory=cuda)
    sampler = DistributedSampler(ds, world, rank, shuffle=True, seed=args.seed)
    loader = DataLoader(ds, args.batch_size, sampler=sampler, num_workers=2, pin_memory=cuda, drop_last=True)
    net = MODELS[args.model](classes)
    graph_kw = {}
    if args.cuda_graphs and cuda and isinstance(getattr(net, "blocks", None), torch.nn.Sequential):
        graph_kw = dict(graph_modules=lambda m: list(m.blocks),
                        graph_sample_inputs=(torch.randn(args.batch_size, 3, 32, 32),))
    trainer = cb.DataParallelTrainer(
        net,
        lambda p: FusedSGD(p, lr=args.lr, momentum=args.momentum, weight_decay=args.weight_decay,
                           nesterov=args.nesterov),
        F.cross_entropy, reducer=args, device=device, autocast_dtype=torch.bfloat16 if (args.bf16 and cuda) else None,
        channels_last=cuda, cudnn_autotune=not args.no_cudnn_autotune, **graph_kw)
    defaults = [round(args.epochs * f) for f in (80 / 150, 120 / 150, 1.0)]
    decay_at = {d if v is None else v for v, d in zip(
        (args.lr_decay_at_epoch1, args.lr_decay_at_epoch2, args.lr_decay_at_epoch3), defaults)}
    stop, log = GracefulStop(), JsonLogger(stdout=True)
    history = []
    result = dict(train_losses=[], test_accuracies=[], time=[], history=history)
    ac_dtype = torch.bfloat16 if (args.bf16 and cuda) else None
    for epoch in range(args.epochs):
        if epoch in decay_at and epoch > 0:
            for group in trainer.optimizer.param_groups:
                group["lr"] /= args.lr_decay_ratio
        sampler.set_epoch(epoch)
        t0, seen, correct, loss_sum = time.time(), 0, 0, 0.0
        for x, y in loader:
            loss = trainer.step(x, y)
            loss_sum += float(loss)
            seen += y.numel()
            if stop.requested:
                break
        dt = time.time() - t0
        rec = dict(epoch=epoch, loss=loss_sum / max(1, len(loader)), img_per_s=seen * world / dt,
                   lr=trainer.optimizer.param_groups[0]["lr"],
                   ef_buffer_mb=(trainer.state.ef_buffer_bytes() / 1e6) if trainer.state else 0.0)
        if rank == 0:       # as the reference: rank 0 evaluates its replica on the whole test set
            rec["test_acc"] = evaluate(trainer.model.module, test_loader, device, ac_dtype, channels_last=cuda)
            result["train_losses"].append(rec["loss"])
            result["test_accuracies"].append(rec["test_acc"])
            result["time"].append(dt)
        history.append(rec)
        log.log(epoch, **rec)
        if stop.requested:
            break
    trainer.check()
    if rank == 0:
        write_results(args, result, world)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
