"""The C++20 host mirror of the reference interface (tensors_b200/host): builds with g++ alone, its
argument checks run without a GPU, and its reference-style known-answer checks run on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "tensors_b200", "host")


def build():
    subprocess.run(["make", "-C", HOST], check=True, capture_output=True)


def test_host_mirror_builds_and_checks_arguments_without_gpu():
    build()
    r = subprocess.run([os.path.join(HOST, "host_test"), "cpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all passed" in r.stdout


@pytest.mark.gpu
def test_host_mirror_known_answers_on_gpu():
    build()
    r = subprocess.run([os.path.join(HOST, "host_test"), "gpu"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "all passed" in r.stdout


@pytest.mark.gpu
def test_training_loop_on_the_host_mirror_learns():
    # Linear -> relu -> Linear -> cross_entropy -> backward -> SGD, all on the device; exits 0 when the
    # loss at least halves
    build()
    r = subprocess.run([os.path.join(HOST, "train_mlp_b200"), "100", "256", "128"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "final_loss" in r.stdout
