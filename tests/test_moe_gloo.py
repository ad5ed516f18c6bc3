"""MoE layers on CPU ranks (expert-parallel and tensor-parallel splits) against a dense loop."""
import torch

from conftest import run_gloo
from moe_common import run_moe_layer


def _ep(rank, world):
    run_moe_layer(rank, world, ep_size=world, dtype=torch.float32, device="cpu")


def _tp(rank, world):
    run_moe_layer(rank, world, ep_size=1, dtype=torch.float32, device="cpu")


def test_moe_layers_expert_parallel_gloo():
    run_gloo(_ep, 2)


def test_moe_layers_tensor_parallel_gloo():
    run_gloo(_tp, 2)
