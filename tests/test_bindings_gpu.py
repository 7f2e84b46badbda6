"""The compiled drop-in boundary: bindings/nts_cuda_stream.cpp implements the reference's cuda/ntsCUDA.hpp
(class Cuda_Stream and the allocation / copy helpers) on libnb_b200.so, and bindings/_build/nts_gpu_harness is the
REFERENCE's own GPU mini-batch code — Sampler::sample_one / load_feature_gpu[_cache] / load_label_gpu, sampCSC's device
mirrors, SingleGPUSampleGraphOp under NtsContext, Parameter::learnC2G_with_decay_Adam — compiled from the reference
tree against that file.  It trains every batch twice, on the GPU through libnb_b200 and on the CPU through the
reference's CPU twin (MiniBatchFuseOp), and exits non-zero unless the two loss curves and the final weights agree
within 1e-3.  The binaries are built by `make -C bindings` where the reference tree exists and travel with the
repository snapshot; where they are absent the test is skipped."""
import os
import re
import subprocess

import numpy as np
import pytest

from test_reference_trainer_cpu import TRAIN, load_train

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HARNESS = os.path.join(ROOT, "bindings", "_build", "nts_gpu_harness")


@pytest.mark.skipif(not os.path.exists(HARNESS), reason="bindings/_build/nts_gpu_harness is built only where the reference tree exists")
@pytest.mark.parametrize("cache_rate", [0.0, 0.3], ids=["zero_copy", "gpu_cache"])
@pytest.mark.parametrize("path", TRAIN, ids=[os.path.basename(p)[:-4] for p in TRAIN])
def test_reference_gpu_classes_on_libnb_b200_match_their_cpu_twin(cuda_device, tmp_path, path, cache_rate):
    g = load_train(path)
    lr, wd = [float(x) for x in g["lr_wd"]]
    g["edges"].astype("<u4").tofile(tmp_path / "g.edge")
    g["feat"].astype("<f4").tofile(tmp_path / "feat.f32")
    g["label"].astype("<i8").tofile(tmp_path / "label.i64")
    g["seeds"].astype("<u4").tofile(tmp_path / "seeds.u32")
    cmd = [HARNESS, str(tmp_path / "g.edge"), str(g["V"]), str(tmp_path / "feat.f32"), str(tmp_path / "label.i64"),
           str(tmp_path / "seeds.u32"), ",".join(map(str, g["fanout"])), "-".join(map(str, g["layers"])), str(g["batch"]),
           str(g["epochs"]), str(lr), str(wd), str(cache_rate)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    text = out.stdout + out.stderr
    assert out.returncode == 0, text[-2000:]
    epochs = re.findall(r"NTSB200 epoch (\d+) loss_gpu ([0-9.]+) loss_cpu ([0-9.]+)", out.stdout)
    assert len(epochs) == g["epochs"]
    for _, lg, lc in epochs:
        assert abs(float(lg) - float(lc)) < 1e-3
    m = re.search(r"NTSB200 batches (\d+) max_loss_diff ([0-9.e+-]+) max_weight_diff ([0-9.e+-]+) cache_nodes (\d+)", out.stdout)
    assert m and int(m.group(1)) == len(g["loss"])
    assert float(m.group(2)) < 1e-3 and float(m.group(3)) < 1e-3
    assert int(m.group(4)) == int(cache_rate * g["V"])
    # the run learns, and lands where the reference's own CPU trainer landed on the same data (other sampled edges)
    first, last = float(epochs[0][1]), float(epochs[-1][1])
    ref_epoch = g["loss"].astype(np.float64).reshape(g["epochs"], -1).mean(axis=1)
    assert last < first - 0.1
    assert abs(last - ref_epoch[-1]) < 0.15


NTS_B200 = os.path.join(ROOT, "bindings", "_build", "nts_b200")


@pytest.mark.skipif(not os.path.exists(NTS_B200), reason="bindings/_build/nts_b200 is built only where the reference tree exists")
@pytest.mark.parametrize("mode,cache,pipelines", [("zerocopy", "CACHE_TYPE:none", 1),
                                                  ("zerocopy", "CACHE_TYPE:rate\nCACHE_RATE:0.3\nCACHE_POLICY:degree", 1),
                                                  ("pipeline", "CACHE_TYPE:rate\nCACHE_RATE:0.25\nCACHE_POLICY:sample", 2),
                                                  ("explicit", "CACHE_TYPE:none", 1)],
                         ids=["zerocopy", "zerocopy_degree_cache", "pipeline_sample_cache", "explicit"])
def test_reference_trainer_class_runs_from_a_cfg_on_libnb_b200(cuda_device, tmp_path, mode, cache, pipelines):
    """bindings/_build/nts_b200 is the reference's GCN_GPU_NEIGHBOR_impl (toolkits/GCN_GPU_NEIGHBOR.hpp), compiled
    unmodified, with every CUDA call landing in libnb_b200.so.  Driven by a .cfg on a small homophilous dataset it must
    print the reference's epoch lines, lower the training loss and classify held-out vertices far above chance."""
    from toy_dataset import write_toy_cfg, write_toy_dataset
    V, F, C = 1500, 16, 4
    base = write_toy_dataset(tmp_path, V, F, C)
    cfg = write_toy_cfg(tmp_path, base, V, F, C, cache=cache, pipelines=pipelines, epochs=8)
    text = cfg.read_text().replace("MODE:zerocopy", "MODE:" + mode)
    cfg.write_text(text)
    out = subprocess.run([NTS_B200, str(cfg)], capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    log = out.stdout + out.stderr
    assert out.returncode == 0, log[-3000:]
    lines = re.findall(r"Epoch (\d+) train_loss ([0-9.]+) train_acc ([0-9.]+) val_loss ([0-9.]+) val_acc ([0-9.]+) "
                       r"test_acc ([0-9.]+)", log)
    assert len(lines) == 8, log[-3000:]
    first, last = float(lines[0][1]), float(lines[-1][1])
    assert last < first
    assert max(float(l[4]) for l in lines) > 0.6      # 4 balanced classes: chance is 0.25
    best = re.search(r"Best-val-acc: ([0-9.]+)", log)
    assert best and float(best.group(1)) > 0.6
