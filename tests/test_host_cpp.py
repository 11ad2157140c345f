"""The C++ host mirror (include/kleos_b200.hpp) and the stand-alone driver built on it
(aristos_b200/csrc/host_driver.cpp, the counterpart of the reference's csrc/main.cu:12-73)."""
import os
import re
import subprocess

import numpy as np
import pytest

from aristos_b200 import build as kbuild, synth
from aristos_b200.config import KleosConfig

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_driver(cfg: KleosConfig, workdir, packed=None, timeout=300):
    """Runs kleos_driver in `workdir` on `cfg`.  With `packed` (fp32 values already rounded to the
    element type) it performs one forward on that image and returns the packed output decoded
    to fp32; without it returns the process result of a timed run."""
    driver = kbuild.build_driver()
    cfg.to_json(os.path.join(workdir, "kleos_config.json"))
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "KLEOS_CONFIG")}
    if packed is None:
        return subprocess.run([driver], cwd=workdir, env=env, capture_output=True, text=True, timeout=timeout)
    src, dst = os.path.join(workdir, "in.bin"), os.path.join(workdir, "out.bin")
    synth.encode(packed, cfg.torch_dtype).tofile(src)
    res = subprocess.run([driver, "--io", src, dst], cwd=workdir, env=env, capture_output=True, text=True,
                         timeout=timeout)
    assert res.returncode == 0, res.stderr
    raw = np.fromfile(dst, dtype=np.float32 if cfg.elem_bytes == 4 else np.uint16)
    return synth.decode(raw, cfg.torch_dtype)


def test_header_compiles_on_its_own(tmp_path):
    src = tmp_path / "t.cpp"
    src.write_text('#include "kleos_b200.hpp"\n'
                   'int main() { kleos::Launch l = kleos::launchFromEnv(); return l.world > 0 ? 0 : 1; }\n')
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-fsyntax-only",
                           "-I", os.path.join(ROOT, "include"), str(src)])


def test_c_abi_header_is_plain_c_and_links(tmp_path):
    """Foreign-function callers (cgo, JNI, ctypes generators) need the header to be C: compile it
    as C11 with warnings as errors, then link a C program against the library and call entry
    points that need no GPU."""
    src = tmp_path / "t.c"
    src.write_text(
        '#include <stdio.h>\n#include <string.h>\n#include "kleos_b200.h"\n'
        'int main(int argc, char** argv) {\n'
        '    kleos_layer_info info;\n'
        '    if (argc != 2) return 2;\n'
        '    if (kleos_config_probe(argv[1], 8, &info) != KLEOS_OK) return 3;\n'
        '    if (kleos_get_rank() != KLEOS_E_STATE) return 4;   /* not initialised */\n'
        '    printf("%d %d %d %lld\\n", info.S, info.EC, info.local_experts, (long long)info.input_elems);\n'
        '    return strlen(kleos_error_string(KLEOS_E_CONFIG)) > 0 ? 0 : 5;\n'
        '}\n')
    exe = tmp_path / "t"
    libdir = os.path.dirname(kbuild.build())
    subprocess.check_call(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic",
                           "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                           "-L", libdir, "-lkleos_b200", f"-Wl,-rpath,{libdir}"])
    cfg = KleosConfig()   # the reference's shipped layer shape
    cfg.to_json(str(tmp_path / "kleos_config.json"))
    out = subprocess.run([str(exe), str(tmp_path / "kleos_config.json")], capture_output=True, text=True,
                         timeout=120)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["8192", "256", "8", str(cfg.input_elems(8))]


def test_driver_fails_loudly_without_a_layer_or_a_gpu(tmp_path):
    driver = kbuild.build_driver()
    res = subprocess.run([driver], cwd=tmp_path, capture_output=True, text=True, timeout=120)
    assert res.returncode == 1 and "kleos_config.json" in res.stderr
    import torch
    if torch.cuda.is_available():
        pytest.skip("the second half needs a machine without a GPU")
    res = run_driver(KleosConfig(sequence_len=128, hidden_size=64, intermediate_size=64, num_experts=4),
                     str(tmp_path))
    assert res.returncode == 1 and "no CUDA device" in res.stderr


def test_driver_rejects_unknown_arguments(tmp_path):
    driver = kbuild.build_driver()
    res = subprocess.run([driver, "--what"], cwd=tmp_path, capture_output=True, text=True, timeout=120)
    assert res.returncode == 2 and "usage" in res.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [2, 0])
def test_driver_forward_matches_the_oracle(tmp_path, dtype):
    """One forward through the C++ mirror (kleos::initialize, moe::forwardHost, kleos::finalize)
    on a seeded packed input, compared with the oracle like every other parity case."""
    from oracle import moe_oracle
    from tests import moe_harness as hz
    cfg = KleosConfig(sequence_len=256, hidden_size=512, intermediate_size=1024, num_experts=8,
                      torch_dtype=dtype)
    packed, views = hz.make_inputs(cfg, 1, bias_scale=0.5)
    ref = moe_oracle.moe_forward(cfg, 1, views)[0]
    o = run_driver(cfg, str(tmp_path), packed[0])
    probs = o[: cfg.S * cfg.PX].reshape(cfg.S, cfg.PX)
    out = o[cfg.S * cfg.PX:].reshape(cfg.S, cfg.H)
    assert np.abs(probs - ref["probs"]).max() <= hz.PROB_TOL[dtype]
    err = np.abs(out - ref["out"]).max() / np.abs(ref["out"]).max()
    assert err <= hz.TOL[dtype], f"driver output error {err}"


@pytest.mark.gpu
def test_driver_timed_run_prints_the_reference_line(tmp_path):
    """Timed mode: the line the reference's driver prints (csrc/main.cu:69)."""
    cfg = KleosConfig(sequence_len=256, hidden_size=512, intermediate_size=1024, num_experts=8)
    res = run_driver(cfg, str(tmp_path))
    assert res.returncode == 0, res.stderr
    m = re.search(r"epRank: 0 took ([0-9.]+)ms", res.stdout)
    assert m and 0.0 < float(m.group(1)) < 50.0, res.stdout


def test_id_rendezvous_between_two_ranks(tmp_path):
    """The C++ mirror hands rank 0's NCCL id to the other ranks through a file.  Two processes
    (no GPU needed: creating the id only loads NCCL) must end up with the same 128 bytes, and a
    rank whose rank 0 never shows up must give up with a message."""
    src = tmp_path / "rv.cpp"
    src.write_text(
        '#include <cstdio>\n#include "kleos_b200.hpp"\n'
        'int main() {\n'
        '    kleos::Launch l = kleos::launchFromEnv();\n'
        '    l.id_timeout_s = 3;\n'
        '    unsigned char id[128] = {};\n'
        '    kleos::exchangeId(l, id);\n'
        '    for (unsigned char c : id) std::printf("%02x", c);\n'
        '    std::printf("\\n");\n'
        '    return 0;\n'
        '}\n')
    exe = tmp_path / "rv"
    libdir = os.path.dirname(kbuild.build())
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                           str(src), "-o", str(exe), "-L", libdir, "-lkleos_b200", f"-Wl,-rpath,{libdir}",
                           "-pthread"])
    idf = str(tmp_path / "id")
    base = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE")}
    procs = [subprocess.Popen([str(exe)], env=dict(base, RANK=str(r), WORLD_SIZE="2", KLEOS_ID_FILE=idf),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for r in (1, 0)]   # the reader starts first and has to wait
    outs = [p.communicate(timeout=120) for p in procs]
    assert all(p.returncode == 0 for p in procs), [o[1] for o in outs]
    ids = [o[0].strip() for o in outs]
    assert len(ids[0]) == 256 and ids[0] == ids[1] and set(ids[0]) != {"0"}
    # a file that an earlier launch left behind (crashed before finalize) is not this launch's id:
    # the reader ignores it until rank 0 has replaced it
    stale = tmp_path / "stale"
    stale.write_bytes(b"\x55" * 128)
    old = os.path.getmtime(stale) - 3600
    os.utime(stale, (old, old))
    procs = [subprocess.Popen([str(exe)], env=dict(base, RANK=str(r), WORLD_SIZE="2", KLEOS_ID_FILE=str(stale)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for r in (1, 0)]
    outs = [p.communicate(timeout=120) for p in procs]
    assert all(p.returncode == 0 for p in procs), [o[1] for o in outs]
    ids = [o[0].strip() for o in outs]
    assert ids[0] == ids[1] and ids[0] != "55" * 128
    os.utime(stale, (old, old))   # rank 0 never shows up again: the old file must not satisfy rank 1
    alone = subprocess.run([str(exe)], env=dict(base, RANK="1", WORLD_SIZE="2", KLEOS_ID_FILE=str(stale)),
                           capture_output=True, text=True, timeout=120)
    assert alone.returncode == 1 and "waited 3 s for the NCCL id" in alone.stderr
    # nobody publishes: rank 1 gives up after its timeout
    lonely = subprocess.run([str(exe)], env=dict(base, RANK="1", WORLD_SIZE="2",
                                                 KLEOS_ID_FILE=str(tmp_path / "never")),
                            capture_output=True, text=True, timeout=120)
    assert lonely.returncode == 1 and "waited 3 s for the NCCL id" in lonely.stderr


@pytest.mark.gpu
def test_driver_two_ranks_through_the_cpp_mirror(tmp_path, gpu_count):
    """Two kleos_driver processes started the way a launcher would (RANK / WORLD_SIZE in the
    environment, the NCCL id through the rendezvous file): both must run the timed forward of
    the reference's shipped layer shape and print the reference's line."""
    if gpu_count < 2:
        pytest.skip("needs 2 GPUs")
    driver = kbuild.build_driver()
    cfg = KleosConfig(sequence_len=2048, hidden_size=1024, intermediate_size=1024, num_experts=16)
    cfg.to_json(os.path.join(tmp_path, "kleos_config.json"))
    base = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "KLEOS_CONFIG")}
    env = dict(base, WORLD_SIZE="2", KLEOS_ID_FILE=str(tmp_path / "id"), KLEOS_WAIT_MS="3000",
               NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([driver], cwd=tmp_path, env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in (0, 1)]
    outs = [p.communicate(timeout=300) for p in procs]
    for r, (p, (so, se)) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, se[-2000:]
        m = re.search(rf"epRank: {r} took ([0-9.]+)ms", so)
        assert m and 0.0 < float(m.group(1)) < 50.0, so
