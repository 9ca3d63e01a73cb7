"""The hand-written protobuf reader and the tokenizer under AddressSanitizer and UndefinedBehaviorSanitizer
(host code only, no GPU): valid files parse, and truncated or corrupted model files and malformed UTF-8 end
in a C++ exception (the reference's std::invalid_argument behaviour), never in an out-of-bounds access.
compute-sanitizer is not available for the device code, so this covers the part that parses untrusted bytes.
"""
import os
import shutil
import subprocess

import numpy as np
import pytest

from cubert_b200 import build as native
from cubert_b200 import frozen_graph, synthetic

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "cubert_b200", "csrc", "host")


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    out = str(tmp_path_factory.mktemp("sanitize") / "host_sanitize")
    cuda_inc = os.path.join(native.CUDA_HOME, "include")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined",
           "-I" + HOST, "-I" + os.path.join(ROOT, "include"), "-I" + cuda_inc,
           os.path.join(ROOT, "tests", "host_sanitize_main.cpp"), os.path.join(HOST, "frozen_graph.cpp"),
           os.path.join(HOST, "tokenizer.cpp"), os.path.join(HOST, "runtime.cpp"),
           "-L" + os.path.join(native.CUDA_HOME, "lib64"), "-lcudart", "-lcublas",
           "-Wl,-rpath," + os.path.join(native.CUDA_HOME, "lib64"), "-o", out]
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, universal_newlines=True)
    if proc.returncode != 0:
        pytest.skip("sanitizer build not possible here: " + proc.stdout[-400:])
    return out


def run(harness, commands):
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    proc = subprocess.run([harness], input=("\n".join(commands) + "\n").encode(), stdout=subprocess.PIPE,
                          stderr=subprocess.PIPE, env=env, timeout=600)
    err = proc.stderr.decode("utf8", errors="replace")    # the tokenizer echoes undecodable input, as the reference does
    assert proc.returncode == 0 and "Sanitizer" not in err and "runtime error" not in err, err[-3000:]
    return proc.stdout.decode("utf8", errors="replace").splitlines()


def test_model_files_valid_truncated_and_corrupted(harness, tmp_path):
    cfg = synthetic.config("tiny")
    var = synthetic.random_weights(cfg, 3)
    good = str(tmp_path / "good.pb")
    frozen_graph.write_frozen_graph(good, var, extra_nodes=["bert/encoder/Reshape", "loss/Softmax"])
    data = open(good, "rb").read()
    lines = run(harness, ["graph float " + good, "graph half " + good])
    assert all(l.startswith("ok %d " % len(var)) for l in lines), lines
    want = sum(float(np.sum(v.astype(np.float64))) for v in var.values())
    assert abs(float(lines[0].split()[2]) - want) < 1e-3 * max(1.0, abs(want))

    rng = np.random.default_rng(0)
    commands = []
    cuts = sorted(set([0, 1, 2, 3, 5, 8, 13, 21, 34, 55, 89] + list(rng.integers(0, len(data), 60)) +
                      [len(data) - k for k in (1, 2, 3, 4, 8, 16)]))
    for i, cut in enumerate(cuts):                        # truncations
        p = str(tmp_path / ("cut%d.pb" % i))
        open(p, "wb").write(data[:cut])
        commands += ["graph float " + p, "graph half " + p]
    for i in range(120):                                  # byte corruption, biased to the framing bytes at the start of nodes
        b = bytearray(data)
        for _ in range(int(rng.integers(1, 6))):
            pos = int(rng.integers(0, min(len(b), 4096))) if rng.random() < 0.5 else int(rng.integers(0, len(b)))
            b[pos] = int(rng.integers(0, 256))
        p = str(tmp_path / ("bad%d.pb" % i))
        open(p, "wb").write(bytes(b))
        commands.append("graph %s %s" % ("half" if i % 2 else "float", p))
    commands.append("graph float " + str(tmp_path / "missing.pb"))
    lines = run(harness, commands)
    assert len(lines) == len(commands)
    assert all(l.startswith("ok ") or l.startswith("rejected: ") for l in lines)
    assert lines[-1].startswith("rejected: ")
    assert sum(l.startswith("rejected") for l in lines) > 20     # truncated files cannot all parse


def test_model_whose_tensor_sizes_disagree_with_its_geometry_is_rejected(harness, tmp_path):
    """A file can parse and still be unusable: shapes that promise more elements than the content holds, a
    sequence length beyond the position table, a head count that does not divide the hidden size, a layer
    count beyond the file's. Each must be refused before a replica copies from the arrays."""
    cfg = synthetic.config("tiny")
    var = synthetic.random_weights(cfg, 3)
    H, L, heads = cfg["hidden"], cfg["layers"], cfg["heads"]
    good = str(tmp_path / "good.pb")
    frozen_graph.write_frozen_graph(good, var)
    commands = ["model float %s 16 %d %d" % (good, L, heads), "model half %s 16 %d %d" % (good, L, heads),
                "model float %s %d %d %d" % (good, cfg["max_position"], L, heads)]
    expect_ok = len(commands)
    # geometry the caller gets wrong
    commands += ["model float %s %d %d %d" % (good, cfg["max_position"] + 1, L, heads),
                 "model float %s 16 %d %d" % (good, L + 1, heads),
                 "model float %s 16 %d %d" % (good, L, heads + 1 if H % (heads + 1) else 7),
                 "model float %s 0 %d %d" % (good, L, heads)]
    # files whose declared shapes and contents disagree
    lies = {
        "vocab": {"bert/embeddings/word_embeddings": (cfg["vocab"] * 4, H)},
        "hidden": {"bert/embeddings/word_embeddings": (cfg["vocab"], H * 2),
                   "bert/embeddings/token_type_embeddings": (cfg["type_vocab"], H * 2)},
        "inter": {"bert/encoder/layer_0/intermediate/dense/bias": (cfg["intermediate"] * 2,)},
        "labels": {"output_weights": (cfg["num_labels"] + 3, H)},
    }
    for name, declared in lies.items():
        p = str(tmp_path / ("lie_%s.pb" % name))
        frozen_graph.write_frozen_graph(p, var, declared_shapes=declared)
        commands.append("model float %s 16 %d %d" % (p, L, heads))
    short = dict(var)
    short["bert/encoder/layer_0/output/dense/kernel"] = var["bert/encoder/layer_0/output/dense/kernel"][:-1]
    p = str(tmp_path / "short.pb")
    frozen_graph.write_frozen_graph(p, short)
    commands.append("model half %s 16 %d %d" % (p, L, heads))
    lines = run(harness, commands)
    assert len(lines) == len(commands)
    assert all(l == "ok" for l in lines[:expect_ok]), lines[:expect_ok]
    assert all(l.startswith("rejected: ") and "invalid" in l for l in lines[expect_ok:]), lines[expect_ok:]


def test_key_extents_and_their_grouping(harness):
    """The host arithmetic behind 'attention over kept keys only': extent = position after the last non-zero mask
    entry, rounded up to the granule, the whole sequence when nothing is kept; sequences counting-sorted by extent."""
    rng = np.random.default_rng(9)
    commands, cases = [], []
    for seq, granule, max_groups, batch in ((128, 32, 16, 37), (128, 8, 16, 5), (512, 64, 16, 64), (40, 32, 16, 9),
                                            (64, 8, 4, 6), (1, 8, 16, 3), (100, 8, 16, 50)):
        lengths = rng.integers(0, seq + 1, batch)
        mask = np.zeros((batch, seq), np.int8)
        for b, n in enumerate(lengths):
            if n > 0:
                mask[b, :n] = rng.integers(-3, 4, n)
                mask[b, n - 1] = rng.choice([-7, 1, 99])         # the last kept key sits at n - 1; holes before it are fine
        cases.append((seq, granule, max_groups, mask, lengths))
        commands.append("extents %d %d %d %s" % (seq, granule, max_groups, mask.tobytes().hex()))
    lines = run(harness, commands)
    assert len(lines) == len(cases)
    for line, (seq, granule, max_groups, mask, lengths) in zip(lines, cases):
        assert line.startswith("ok "), line
        parts = [p.split() for p in line[3:].split("|")]
        extents = np.array(parts[0], int)
        want = np.where(lengths == 0, seq, np.minimum((lengths + granule - 1) // granule * granule, seq))
        assert np.array_equal(extents, want), (seq, granule)
        order, start, group_extent = (np.array(p[1:], int) for p in parts[1:4])
        buckets = (seq + granule - 1) // granule
        if buckets > max_groups:
            assert order.size == 0 and group_extent.size == 0       # too many distinct extents: no grouping
            continue
        assert sorted(order.tolist()) == list(range(len(lengths)))            # a permutation
        assert np.all(np.diff(extents[order]) >= 0)                           # growing extent
        assert start[0] == 0 and start[-1] == len(lengths) and np.all(np.diff(start) > 0)
        for g, e in enumerate(group_extent):
            assert np.all(extents[order[start[g]:start[g + 1]]] == e)
        assert np.all(np.diff(group_extent) > 0)


def test_tokenizer_on_valid_and_malformed_text(harness, tmp_path):
    vocab = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "hello", "world", "##s", "un", "##aff", "##able", "!", ",", "中", "文",
             "e", "cafe", "é"]
    vp = str(tmp_path / "vocab.txt")
    open(vp, "w", encoding="utf8").write("\n".join(vocab) + "\n")
    texts = [b"hello worlds!", "Café 中文, unaffable".encode("utf8"), b"", b" \t\n ", b"a" * 5000,
             "\U0001f600 emoji ́́".encode("utf8"),
             b"\xff\xfe bad start", b"trunc \xe4\xb8", b"overlong \xc0\xaf", b"lone \x80 cont", b"\xf4\x90\x80\x80 too big",
             b"\xed\xa0\x80 surrogate", bytes(range(1, 128)), bytes([0xe4, 0xb8, 0xad] * 700)]
    rng = np.random.default_rng(1)
    texts += [bytes(rng.integers(1, 256, size=int(rng.integers(1, 300)), dtype=np.uint8)) for _ in range(150)]
    commands = []
    for i, t in enumerate(texts):
        t = t.replace(b"\x00", b" ")
        commands.append("tok %d %s %d %s" % (i % 2, vp, [8, 16, 128][i % 3], t.hex() or "20"))
    lines = run(harness, commands)
    assert len(lines) == len(commands)
    assert all(l.startswith("ok ") or l.startswith("rejected: ") for l in lines)
    first = [int(x) for x in lines[0].split()[1:]]
    assert first[:6] == [2, 4, 5, 6, 10, 3] and set(first[6:]) == {0}     # [CLS] hello world ##s ! [SEP] pad...
