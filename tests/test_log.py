"""The leveled logger: threshold, format, and that the engine's lines come through it."""
import re

from tffinfer_b200 import log


def test_levels_and_format(capsys):
    old = log.get_level()
    try:
        log.set_level("info")
        log.debug("not shown %d", 1)
        log.info("pages: %d of %d", 3, 8)
        log.warning("plain text with a % sign")      # no arguments: taken as it is
        err = capsys.readouterr().err.splitlines()
        assert len(err) == 2
        assert re.fullmatch(r"\[tffinfer_b200 INFO \+\d+\.\d{3}s\] pages: 3 of 8", err[0])
        assert err[1].endswith("plain text with a % sign") and "WARNING" in err[1]
        log.set_level("error")
        log.warning("hidden")
        log.error("shown")
        assert capsys.readouterr().err.count("\n") == 1
        log.set_level("off")
        log.error("hidden too")
        assert capsys.readouterr().err == ""
        try:
            log.set_level("loud")
            assert False
        except ValueError as e:
            assert "loud" in str(e)
    finally:
        log.set_level(old)


def test_the_engine_reports_its_cache_and_a_refused_request(tmp_path, capsys):
    from cpu_ops import CpuOps
    from helpers import make_model_dir
    from tffinfer_b200.config import EngineConfig
    from tffinfer_b200.engine import Engine, ModelRunner
    old = log.get_level()
    try:
        log.set_level("info")
        d = make_model_dir(tmp_path, "C")
        eng = Engine(runner=ModelRunner(d, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=64, device="cpu",
                                                        max_live_requests=2), ops=CpuOps()))
        err = capsys.readouterr().err
        assert "cache group 0" in err and "cache group 1" in err and "window 24" in err and "all keys" in err
        assert "4 layers" in err
        out = eng.generate([list(range(1, 100))], max_new_tokens=2)      # 99 tokens into a pool of 64
        assert out == [[]]
        assert "out_of_memory" in capsys.readouterr().err
    finally:
        log.set_level(old)
