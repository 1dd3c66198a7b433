"""Training demo of the binary layers: the three-hidden-layer MLP of the reference's tests/python/test_model_demo.py
(:120-151) with the same optimiser groups, loss and loop (:29-73, :186-230), on the layers of bgemm_linear.py.

Forward passes of the binary layers run on the sm_100a kernels; backward passes are the reference's
straight-through / Bi-Real / elastic formulas in torch. The reference trains on `unsw_nb15_binarized.npz`,
which it does not ship; pass its directory with --data-dir to use it (same slicing as :89-101: the first 512
columns minus 0.5 as inputs, the last column as the label, sample count rounded down to a multiple of 32).
Without --data-dir a seeded synthetic stand-in of the same shape is used: 512 random bits per sample, label =
whether a fixed random hyperplane over a 64-bit subset is crossed (learnable, not trivially so).

    python train_demo.py {bgemm_elastic,bgemm_bireal,nn_elastic,bnn_fp16,fp16} [--epochs E] [--data-dir DIR]
"""
from __future__ import annotations

import argparse
import time

import numpy as np
import torch
import torch.nn as nn
from torch.utils.data import DataLoader, TensorDataset

from bgemm_linear import BGEMMLinear, BGEMMLinear_bireal, BGEMMLinear_elastic_signed, BNNLinear, NNLinear_elastic_signed

LAYERS = {
    "bgemm_elastic": BGEMMLinear_elastic_signed,
    "nn_elastic": NNLinear_elastic_signed,
    "bgemm_bireal": BGEMMLinear_bireal,
    "bgemm": BGEMMLinear,
    "bnn_fp16": BNNLinear,
    "fp16": nn.Linear,
}
SCALING_FACTORS = ("sw", "sa", "zpw", "zpa")


class FC_half2float(nn.Linear):
    """Final classifier in fp32 whatever the dtype of the features (test_model_demo.py:106-117)."""

    def __init__(self, in_channels, out_channels, bias=False):
        super().__init__(in_channels, out_channels, bias)

    def forward(self, x):
        out = nn.functional.linear(x.float(), self.weight.float())
        if self.bias is not None:
            out = out + self.bias.view(1, -1).expand_as(out)
        return out


class MLP(nn.Module):
    """Linear -> (BN, dropout, ReLU) -> binary -> (...) -> binary -> (...) -> fp32 classifier."""

    def __init__(self, Linear=BGEMMLinear, bias=True, input_size=512, hidden1=128, hidden2=128, hidden3=128, num_classes=1, dropout=0.5):
        super().__init__()
        self.lin1 = nn.Linear(input_size, hidden1, bias=bias)
        self.lin2 = Linear(hidden1, hidden2, bias=bias)
        self.lin3 = Linear(hidden2, hidden3, bias=bias)
        self.relu = nn.ReLU()
        self.dropout = nn.Dropout(dropout)
        self.bn1, self.bn2, self.bn3 = nn.BatchNorm1d(hidden1), nn.BatchNorm1d(hidden2), nn.BatchNorm1d(hidden3)
        self.fc = FC_half2float(hidden3, num_classes, bias=True)

    def forward(self, x):
        x = self.relu(self.dropout(self.bn1(self.lin1(x))))
        x = self.relu(self.dropout(self.bn2(self.lin2(x))))
        x = self.relu(self.dropout(self.bn3(self.lin3(x))))
        return self.fc(x)


def synthetic_dataset(samples: int, seed: int, features: int = 512) -> TensorDataset:
    """Seeded stand-in for the binarised intrusion-detection table: {0,1} features minus 0.5, one binary label."""
    g = torch.Generator().manual_seed(1234)                     # the labelling rule is the same for every split
    subset = torch.randperm(features, generator=g)[:64]
    plane = torch.randn(64, generator=g)
    g = torch.Generator().manual_seed(seed)
    bits = torch.randint(0, 2, (samples // 32 * 32, features), generator=g).float()
    label = ((bits[:, subset] - 0.5) @ plane > 0).float()
    return TensorDataset(bits - 0.5, label)


def file_dataset(data_dir: str, train: bool) -> TensorDataset:
    table = np.load(data_dir + "/unsw_nb15_binarized.npz")["train" if train else "test"].astype(np.float16)
    table = torch.from_numpy(table)
    n = table.shape[0] // 32 * 32
    return TensorDataset(table[:n, :512] - 0.5, table[:n, -1])


def make_optimizer(model: nn.Module, lr: float = 1e-3):
    """Adam with the quantisation scales in their own 1e-4 group (test_model_demo.py:200-206). As in the reference,
    scales that a layer creates on its first batch join only if the optimiser is built after that batch."""
    named = list(model.named_parameters())
    groups = [
        {"params": [p for n, p in named if any(s in n for s in SCALING_FACTORS)], "lr": 1e-4},
        {"params": [p for n, p in named if not any(s in n for s in SCALING_FACTORS)]},
    ]
    return torch.optim.Adam(groups, lr=lr, betas=(0.9, 0.999))


def train_epoch(model, loader, optimizer, criterion, device, dtype=torch.float):
    model.train()
    losses = []
    for inputs, target in loader:
        inputs, target = inputs.to(device), target.to(device)
        optimizer.zero_grad()
        loss = criterion(model(inputs.to(dtype)), target.to(torch.float).unsqueeze(1))
        loss.backward()
        optimizer.step()
        losses.append(float(loss.detach()))
    return losses


@torch.no_grad()
def accuracy(model, loader, device, dtype=torch.float) -> float:
    model.eval()
    hit = total = 0
    for inputs, target in loader:
        pred = torch.sigmoid(model(inputs.to(device).to(dtype))).reshape(-1) > 0.5
        hit += int((pred.cpu() == (target > 0.5)).sum())
        total += target.numel()
    return hit / max(total, 1)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("model", nargs="?", default="bgemm_elastic", choices=sorted(LAYERS))
    ap.add_argument("--epochs", type=int, default=20)
    ap.add_argument("--batch-size", type=int, default=256)
    ap.add_argument("--data-dir", default=None)
    ap.add_argument("--samples", type=int, default=32768, help="synthetic training samples")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("the binary layers run on the GPU only")
    device = torch.device("cuda")
    torch.manual_seed(0)
    np.random.seed(0)
    model = MLP(Linear=LAYERS[args.model], bias=True).to(device)
    if args.data_dir:
        train_set, test_set = file_dataset(args.data_dir, True), file_dataset(args.data_dir, False)
    else:
        train_set, test_set = synthetic_dataset(args.samples, 1), synthetic_dataset(args.samples // 4, 2)
    # drop_last: the last, smaller batch would otherwise reach the layers with a row count the reference forbids
    train_loader = DataLoader(train_set, batch_size=args.batch_size, shuffle=True, drop_last=True)
    test_loader = DataLoader(test_set, batch_size=args.batch_size, shuffle=False)
    criterion = nn.BCEWithLogitsLoss().to(device)
    optimizer = make_optimizer(model)
    t0 = time.time()
    for epoch in range(args.epochs):
        losses = train_epoch(model, train_loader, optimizer, criterion, device)
        print("epoch %d  training loss = %f  test accuracy = %f" % (epoch, float(np.mean(losses)), accuracy(model, test_loader, device)))
    print("Total training time: %.5f s" % (time.time() - t0))


if __name__ == "__main__":
    main()
