"""The library's logger namespace and its environment switch (PTB200_VERBOSITY)."""
import logging
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import sys
sys.path.insert(0, sys.argv[1])
import pytorch_transformers_b200 as ptb
from pytorch_transformers_b200.utils import logging as log
cfg = ptb.FalconConfig.from_dict({"hidden_size": 64, "num_attention_heads": 4, "some_new_key": 5, "another": [1]})
assert cfg.extra == {"some_new_key": 5, "another": [1]}
print("level", log.get_verbosity())
"""


def run(level=None):
    env = {k: v for k, v in os.environ.items() if k != "PTB200_VERBOSITY"}
    if level is not None:
        env["PTB200_VERBOSITY"] = level
    return subprocess.run([sys.executable, "-c", SCRIPT, ROOT], capture_output=True, text=True, env=env, timeout=120)


def test_unknown_config_keys_are_kept_and_named_at_debug_level():
    quiet = run()
    assert quiet.returncode == 0, quiet.stderr
    assert f"level {logging.WARNING}" in quiet.stdout and "some_new_key" not in quiet.stderr
    loud = run("debug")
    assert loud.returncode == 0, loud.stderr
    assert f"level {logging.DEBUG}" in loud.stdout
    line = [ln for ln in loud.stderr.splitlines() if "some_new_key" in ln]
    assert line and "another" in line[0] and line[0].startswith("[pytorch_transformers_b200.config.base]")


def test_an_unknown_level_is_reported_and_the_default_kept():
    odd = run("chatty")
    assert odd.returncode == 0 and f"level {logging.WARNING}" in odd.stdout
    assert "PTB200_VERBOSITY" in odd.stderr


def test_every_module_logs_under_one_namespace():
    from pytorch_transformers_b200.utils import logging as log
    a = log.get_logger("pytorch_transformers_b200.weights.loader")
    b = log.get_logger("somewhere.else")
    root = log.get_logger()
    assert a.parent is not None and a.name.startswith(root.name + ".") and b.name.startswith(root.name + ".")
    assert root.propagate is False and len(root.handlers) >= 1
    before = log.get_verbosity()
    try:
        log.set_verbosity("error")
        assert not a.isEnabledFor(logging.WARNING) and a.isEnabledFor(logging.ERROR)
    finally:
        log.set_verbosity(before)
