"""The C interface (capi/engine.h): called through its exported C symbols with ctypes, and from a C program of its
own (tests/capi_example.c) that links the library and libpython. The tokens are the Python entry point's: there is
one engine behind both. After an error a call returns a status and the next call works (the reference:
tests/test_errors.c:33-126)."""
import ctypes
import os
import shutil
import subprocess
import sys
import sysconfig

import pytest
import torch

from tiny import TINY, random_tokens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class Request(ctypes.Structure):
    _fields_ = [("tokens", ctypes.POINTER(ctypes.c_int32)), ("n", ctypes.c_int32)]


TOKEN_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32)
STOP_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)


class Sink(ctypes.Structure):
    _fields_ = [("ctx", ctypes.c_void_p), ("token", TOKEN_FN), ("stop", STOP_FN)]


class Options(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_char_p), ("context", ctypes.c_int32), ("batch", ctypes.c_int32),
                ("step_tokens", ctypes.c_int32), ("kernels", ctypes.c_char_p), ("package_root", ctypes.c_char_p)]


class Generation(ctypes.Structure):
    _fields_ = [("tokens", ctypes.c_int32), ("temperature", ctypes.c_float), ("top_k", ctypes.c_int32),
                ("top_p", ctypes.c_float), ("seed", ctypes.c_uint32), ("stop_ids", ctypes.POINTER(ctypes.c_int32)),
                ("n_stop_ids", ctypes.c_int32)]


def _library():
    from smolmoe_c99_b200.capi import build
    lib = ctypes.CDLL(build())
    lib.lm_open.restype = ctypes.c_void_p
    lib.lm_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(Options), ctypes.c_char_p]
    lib.lm_close.argtypes = [ctypes.c_void_p]
    lib.lm_generate.argtypes = [ctypes.c_void_p, ctypes.POINTER(Request), ctypes.c_int32, ctypes.POINTER(Generation), ctypes.POINTER(Sink)]
    lib.lm_slot_alloc.argtypes = [ctypes.c_void_p]
    lib.lm_slot_free.argtypes = [ctypes.c_void_p, ctypes.c_int32]
    lib.lm_slot_length.argtypes = [ctypes.c_void_p, ctypes.c_int32]
    lib.lm_step.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32), ctypes.c_int32,
                            ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_uint8), ctypes.POINTER(ctypes.c_float)]
    lib.lm_last_error.restype = ctypes.c_char_p
    return lib


def test_the_library_builds_and_refuses_without_a_gpu(tmp_path):
    """No GPU is needed to be turned away: a folder that is not there, an unknown dtype."""
    lib = _library()
    err = ctypes.create_string_buffer(512)
    assert lib.lm_open(str(tmp_path / "nowhere").encode(), None, err) is None
    assert err.value and lib.lm_last_error() == err.value
    options = Options(b"float16", 0, 0, 0, None, None)
    assert lib.lm_open(str(tmp_path / "nowhere").encode(), ctypes.byref(options), err) is None
    assert lib.lm_generate(None, None, 0, None, None) == -1 and b"request" in lib.lm_last_error()
    assert lib.lm_slot_alloc(None) == -1 and b"not open" in lib.lm_last_error()


@pytest.mark.gpu
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_generate_and_step_through_the_c_symbols(model_dirs, name, dtype):
    from smolmoe_c99_b200 import Model
    lib = _library()
    err = ctypes.create_string_buffer(512)
    options = Options(dtype.encode(), 96, 3, 0, b"fast", None)
    model = lib.lm_open(model_dirs[name].encode(), ctypes.byref(options), err)
    assert model, err.value
    vocab = TINY[name]["vocab_size"]
    prompts = [random_tokens(n, vocab, 900 + n) for n in (5, 11, 17, 2)]       # four requests, batches of three
    arrays = [(ctypes.c_int32 * len(p))(*p) for p in prompts]
    requests = (Request * len(prompts))(*[Request(a, len(a)) for a in arrays])
    reference = Model.from_folder(model_dirs[name], dtype, context=96, batch=3)
    for temperature, seed in ((0.0, 1), (0.8, 7)):
        got, lasts = {i: [] for i in range(len(prompts))}, []

        def on_token(ctx, request, token, last):
            got[request].append(token)
            if last:
                lasts.append(request)

        sink = Sink(None, TOKEN_FN(on_token), STOP_FN(0))
        generation = Generation(8, temperature, 40, 0.95, seed, None, 0)
        assert lib.lm_generate(model, requests, len(prompts), ctypes.byref(generation), ctypes.byref(sink)) == 0, lib.lm_last_error()
        want = reference.generate(prompts, tokens=8, temperature=temperature, top_k=40, top_p=0.95, seed=seed, stop_ids=(), batch=3)
        assert [got[i] for i in range(len(prompts))] == want
        assert sorted(lasts) == list(range(len(prompts)))
    # the sink can end a generation: nothing after the step in which it said so
    seen = []
    sink = Sink(None, TOKEN_FN(lambda ctx, r, t, last: seen.append(r)), STOP_FN(lambda ctx: 1))
    assert lib.lm_generate(model, requests, 1, ctypes.byref(Generation(8, 0.0, 0, 0.0, 0, None, 0)), ctypes.byref(sink)) == 0
    assert seen == [0]
    # the step function, and errors that leave the model usable
    slot = lib.lm_slot_alloc(model)
    assert slot >= 0
    toks = (ctypes.c_int32 * 5)(*prompts[0])
    logits = (ctypes.c_float * vocab)()
    one = (ctypes.c_int32 * 1)
    assert lib.lm_step(model, one(slot), one(5), 1, toks, (ctypes.c_uint8 * 1)(1), logits) == 0, lib.lm_last_error()
    engine = reference.engine
    s = engine.open_sequence()
    want_row = engine.step([s], [prompts[0]]).cpu()[0]
    engine.close_sequence(s)
    assert torch.equal(torch.tensor(list(logits)), want_row) if dtype == "float32" else \
        float((torch.tensor(list(logits)) - want_row).abs().max()) == 0.0
    assert lib.lm_slot_length(model, slot) == 5
    assert lib.lm_step(model, one(slot), one(1), 1, one(vocab), None, None) == -1 and b"out of vocabulary" in lib.lm_last_error()
    assert lib.lm_step(model, one(77), one(1), 1, one(1), None, None) == -1 and b"not open" in lib.lm_last_error()
    assert lib.lm_slot_length(model, slot) == 5                       # the refused steps changed nothing
    assert lib.lm_step(model, one(slot), one(1), 1, one(3), (ctypes.c_uint8 * 1)(0), None) == 0 and lib.lm_slot_length(model, slot) == 6
    assert lib.lm_slot_free(model, slot) == 0 and lib.lm_slot_free(model, slot) != 0
    lib.lm_close(model)


@pytest.mark.gpu
def test_a_c_program_over_the_interface(model_dirs, tmp_path):
    """tests/capi_example.c, compiled here against engine.h, the library and libpython, run as a process of its own."""
    from smolmoe_c99_b200 import Model
    from smolmoe_c99_b200.capi import build, header
    cc = shutil.which("cc") or shutil.which("gcc")
    libdir, ldlib = sysconfig.get_config_var("LIBDIR"), sysconfig.get_config_var("LDLIBRARY") or ""
    if not cc or not ldlib.endswith(".so") or not os.path.exists(os.path.join(libdir, ldlib)):
        pytest.skip("no C compiler or no shared libpython on this machine")
    lib = build()
    exe = str(tmp_path / "capi_example")
    name = ldlib[3:-3]
    made = subprocess.run([cc, "-O1", "-std=c11", "-I", os.path.dirname(header()), os.path.join(ROOT, "tests", "capi_example.c"),
                           "-o", exe, lib, f"-L{libdir}", f"-l{name}", f"-Wl,-rpath,{os.path.dirname(lib)}", f"-Wl,-rpath,{libdir}"],
                          capture_output=True, text=True)
    assert made.returncode == 0, made.stderr
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([ROOT] + [p for p in sys.path if p.endswith("site-packages")]))
    run = subprocess.run([exe, model_dirs["A"]], capture_output=True, text=True, env=env, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = run.stdout.strip().splitlines()
    assert lines[0] == f"vocab 256 context 128 layers 2"
    want = Model.from_folder(model_dirs["A"], "float32", context=128, batch=4).generate([[5, 17, 3, 99, 42], [7, 7, 1]], tokens=6, stop_ids=())
    assert lines[1] == "generated 0: " + " ".join(map(str, want[0])) and lines[2] == "generated 1: " + " ".join(map(str, want[1]))
    assert lines[3] == f"step argmax {want[0][0]} length 5" and lines[4].startswith("refused: token 256 out of vocabulary")
