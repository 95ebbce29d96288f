"""The package's public names (no GPU)."""
import subprocess
import sys

import pytest

from tests.util import ROOT


def test_every_exported_name_resolves():
    import llmgen_b200
    for name in llmgen_b200._EXPORTS:
        assert getattr(llmgen_b200, name).__name__ == name
        assert name in dir(llmgen_b200)
    with pytest.raises(AttributeError, match="no attribute 'EngineConfig'"):
        llmgen_b200.EngineConfig


def test_import_and_workload_command_do_not_load_torch():
    code = ("import sys, llmgen_b200, llmgen_b200.workload; "
            "sys.exit(1 if 'torch' in sys.modules else 0)")
    assert subprocess.run([sys.executable, "-c", code], cwd=ROOT, timeout=300).returncode == 0
