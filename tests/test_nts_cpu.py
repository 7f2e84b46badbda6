"""Host logic of the cfg-driven entry: cfg parser (core/GraphSegment.cpp:196-405 semantics), the
reference's text input formats, the epoch log line.  No GPU needed."""
import re

import numpy as np

from neutronbench_b200.nts import InputInfo, epoch_log_line, random_generate, read_feature_label_mask


def _parse_num(line, mode):
    """The reference's log scraper (exp/utils.py:13-24): first number after the keyword."""
    return float(re.findall(r"\d+\.?\d*", line[line.find(mode):])[0])


def test_cfg_parser_last_wins_comments_unknown(tmp_path, capsys):
    cfg = tmp_path / "a.cfg"
    cfg.write_text("# comment\nALGORITHM:GCNNEIGHBORGPU\nALGORITHM:GCNNEIGHBORGPUEXP3\nALGORITHM:GCNNEIGHBORGPU\n"
                   "VERTICES:169343\nLAYERS:128-128-40\nFANOUT:10,25\nVALFANOUT:10-25\nBATCH_SIZE:128\n"
                   "BATCH_SIZE:1024\nEDGE_FILE:./data/ogbn-arxiv/ogbn-arxiv.edge\nFEATURE_FILE:random\n\n"
                   "CACHE_TYPE:rate\nCACHE_RATE:0.2\nCACHE_POLICY:degree\nMODE:zerocopy\nLEARN_RATE:0.01\n"
                   "WEIGHT_DECAY:0.0001\nDROP_RATE:0.5\nEPOCHS:3\nPROC_CUDA:0\nNOT_A_KEY:1\nRUN_TIME:300\n")
    info = InputInfo().readFromCfgFile(str(cfg))
    assert info.algorithm == "GCNNEIGHBORGPU" and info.vertices == 169343 and info.batch_size == 1024
    assert info.layers() == [128, 128, 40]
    assert info.fanout_hop_order() == [25, 10]          # cfg lists layer order; the sampler gets seeds first
    assert info.val_fanout_hop_order() == [25, 10]      # dash-separated lists are accepted too
    assert info.dataset_name == "ogbn-arxiv"
    assert info.cache_type == "rate" and abs(info.cache_rate - 0.2) < 1e-9 and info.run_time == 300
    assert info.unknown == ["NOT_A_KEY"]
    assert "not supported configure NOT_A_KEY" in capsys.readouterr().out


def test_text_readers(tmp_path):
    V, F = 5, 3
    (tmp_path / "g.feat").write_text("".join(f"{i} {i}.5 {i + 1} -{i}\n" for i in range(V)))
    (tmp_path / "g.label").write_text("".join(f"{i} {i % 2}\n" for i in range(V)))
    (tmp_path / "g.mask").write_text("0 train\n1 val\n2 eval\n3 test\n4 unknown\n")
    feat, label, mask = read_feature_label_mask(str(tmp_path / "g.feat"), str(tmp_path / "g.label"),
                                                str(tmp_path / "g.mask"), V, F)
    np.testing.assert_allclose(feat[3], [3.5, 4.0, -3.0])
    np.testing.assert_array_equal(label, [0, 1, 0, 1, 0])
    np.testing.assert_array_equal(mask, [0, 1, 1, 2, 3])


def test_random_generate_split():
    feat, label, mask = random_generate(1000, 8, 7)
    assert (feat == 1.0).all() and label.min() >= 0 and label.max() < 7
    assert (mask == 0).sum() == 650 and (mask == 1).sum() == 100 and (mask == 2).sum() == 250


def test_epoch_line_is_parseable_by_the_reference_scraper():
    line = epoch_log_line(7, 1.234, 0.5, 1.5, 0.625, 0.75, 0.321, 0.1, 0.05, 0.06, 0.07, 0.2, 3.21, 1024, 5000)
    assert line.startswith("Epoch 007 train_loss 1.234 train_acc 0.500")
    assert _parse_num(line, "val_acc") == 0.625
    assert _parse_num(line, "train_time") == 0.321
    assert _parse_num(line, "gcn_run_time") == 3.21


def test_feature_sidecar_round_trip(tmp_path):
    from neutronbench_b200.nts import feature_sidecar_path, read_feature
    V, F = 40, 5
    rng = np.random.RandomState(0)
    feat = rng.randn(V, F).astype(np.float32)
    path = tmp_path / "toy.feat"
    with open(path, "w") as f:
        for i in rng.permutation(V):                      # any line order; ids outside the graph are ignored
            f.write(f"{i} " + " ".join(repr(float(x)) for x in feat[i]) + "\n")
        f.write(f"{V + 3} " + " ".join("1.0" for _ in range(F)) + "\n")
    first = read_feature(str(path), V, F)
    np.testing.assert_array_equal(first, feat)
    side = feature_sidecar_path(str(path), V, F)
    import os
    assert os.path.getsize(side) == 4 * V * F
    np.testing.assert_array_equal(read_feature(str(path), V, F), feat)          # second read: from the side-car
    np.testing.assert_array_equal(np.fromfile(side, dtype="<f4").reshape(V, F), feat)
    # a stale or wrong-sized side-car is not trusted
    with open(side, "wb") as f:
        f.write(b"\0" * 12)
    np.testing.assert_array_equal(read_feature(str(path), V, F), feat)
    np.testing.assert_array_equal(read_feature(str(path), V, F, use_sidecar=False), feat)


def test_multi_label_file_format(tmp_path):
    """CLASSES > 1: label lines are "id count idx..." and become multi-hot rows (core/ntsDataloador.hpp:304-312)."""
    V, F, C = 6, 2, 5
    (tmp_path / "f").write_text("".join(f"{i} 0.5 1.5\n" for i in range(V)))
    (tmp_path / "l").write_text("0 2 1 4\n1 0\n2 1 0\n3 3 0 2 4\n5 1 3\n")
    (tmp_path / "m").write_text("".join(f"{i} train\n" for i in range(V)))
    feat, label, mask = read_feature_label_mask(str(tmp_path / "f"), str(tmp_path / "l"), str(tmp_path / "m"), V, F, C)
    want = np.zeros((V, C), np.int64)
    want[0, [1, 4]] = 1
    want[2, 0] = 1
    want[3, [0, 2, 4]] = 1
    want[5, 3] = 1
    np.testing.assert_array_equal(label, want)
    assert feat.shape == (V, F) and (mask == 0).all()
