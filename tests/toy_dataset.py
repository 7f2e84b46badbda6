"""A small homophilous dataset written in the reference's file formats (binary edge list of u32 pairs; text feature,
label and mask tables keyed by vertex id, core/ntsDataloador.hpp:264-345) plus a GCNNEIGHBORGPU .cfg."""
import numpy as np

from neutronbench_b200 import synth


def write_toy_dataset(root, V=1500, F=16, C=4, E=30000, seed=0):
    """Returns the path stem; files are <stem>.edge/.feat/.label/.mask."""
    rng = np.random.RandomState(seed)
    label = rng.randint(0, C, V)
    # most edges stay inside a class, so a GCN can learn it
    src = rng.randint(0, V, E)
    same = rng.rand(E) < 0.9
    pools = [np.nonzero(label == c)[0] for c in range(C)]
    dst = np.where(same, np.array([pools[label[s]][rng.randint(len(pools[label[s]]))] for s in src]),
                   rng.randint(0, V, E))
    loops = np.arange(V)
    edges = np.stack([np.concatenate([src, dst, loops]), np.concatenate([dst, src, loops])], axis=1).astype("<u4")
    (root / "data" / "toy").mkdir(parents=True)
    base = root / "data" / "toy" / "toy"
    edges.tofile(str(base) + ".edge")
    feat = np.eye(C)[label] + 0.5 * rng.randn(V, C)
    feat = np.concatenate([feat, rng.randn(V, F - C)], axis=1)
    with open(str(base) + ".feat", "w") as f:
        for i in range(V):
            f.write(str(i) + " " + " ".join(f"{x:.5f}" for x in feat[i]) + "\n")
    with open(str(base) + ".label", "w") as f:
        f.writelines(f"{i} {label[i]}\n" for i in range(V))
    mask = synth.split_mask(V, 1)
    names = {0: "train", 1: "val", 2: "test"}
    with open(str(base) + ".mask", "w") as f:
        f.writelines(f"{i} {names[int(mask[i])]}\n" for i in range(V))
    return base


def write_toy_cfg(root, base, V=1500, F=16, C=4, cache="CACHE_TYPE:none", pipelines=1, epochs=8, extra=""):
    cfg = root / "toy.cfg"
    cfg.write_text(f"ALGORITHM:GCNNEIGHBORGPU\nVERTICES:{V}\nLAYERS:{F}-32-{C}\nFANOUT:5,10\nVALFANOUT:5,10\n"
                   f"BATCH_SIZE:256\nBATCH_TYPE:shuffle\nEPOCHS:{epochs}\nEDGE_FILE:{base}.edge\n"
                   f"FEATURE_FILE:{base}.feat\nLABEL_FILE:{base}.label\nMASK_FILE:{base}.mask\nMODE:zerocopy\n{cache}\n"
                   f"PIPELINES:{pipelines}\nLEARN_RATE:0.01\nWEIGHT_DECAY:0.0001\nDROP_RATE:0.1\nBATCH_NORM:0\n{extra}")
    return cfg
