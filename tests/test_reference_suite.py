"""The reference's own CPU unit tests, run against THIS package.

Where a copy of the reference's ``tests/`` tree is available (``baseline/_ref_tests``, or the
directory named by ``DASER_REFERENCE_TESTS``), its server, retrieval, position, config and RPC
client tests are run in a child pytest with the package name ``daser`` aliased to ``daser_b200``:
same constructors, same methods, same wire behaviour.  Skipped elsewhere.

The child's conftest adds what the reference's suite expects from its environment: the
``asyncio`` marker (it relies on pytest-asyncio, which is not required here), an event loop for
its synchronous tests that call ``asyncio.get_event_loop()``, and the private helper name
``_hash_tokens`` its tests import from the prefix index module.
"""

import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.environ.get("DASER_REFERENCE_TESTS") or os.path.join(ROOT, "baseline", "_ref_tests")
pytestmark = pytest.mark.slow

CONFTEST = '''
import asyncio, importlib, inspect, sys
import pytest
sys.path.insert(0, {root!r})
for name in ("", ".config", ".logging", ".server", ".server.chunk_manager", ".server.metadata_store",
             ".server.doc_registry", ".server.ipc_server", ".server.__main__", ".retrieval", ".retrieval.base",
             ".retrieval.prefix", ".position", ".position.base", ".position.fixed_offset", ".connector",
             ".connector.ipc_client", ".service", ".service.chunker"):
    sys.modules["daser" + name] = importlib.import_module("daser_b200" + name)
from daser_b200.hashing import hash_tokens
sys.modules["daser.retrieval.prefix"]._hash_tokens = hash_tokens

def pytest_configure(config):
    config.addinivalue_line("markers", "asyncio: run the coroutine with asyncio.run")

@pytest.hookimpl(tryfirst=True)
def pytest_pyfunc_call(pyfuncitem):
    if inspect.iscoroutinefunction(pyfuncitem.obj):
        kwargs = {{a: pyfuncitem.funcargs[a] for a in pyfuncitem._fixtureinfo.argnames}}
        asyncio.run(pyfuncitem.obj(**kwargs))
        return True

@pytest.fixture(autouse=True)
def _event_loop_for_sync_tests():
    loop = asyncio.new_event_loop()
    asyncio.set_event_loop(loop)
    yield
    loop.close()
    asyncio.set_event_loop(None)
'''


@pytest.mark.skipif(not os.path.isdir(SRC), reason="no copy of the reference's tests on this machine")
def test_reference_unit_tests_pass_against_this_package(tmp_path):
    work = tmp_path / "ref_tests"
    work.mkdir()
    picked = 0
    for name in ("server", "retrieval", "position", "test_config.py"):
        src = os.path.join(SRC, name)
        if os.path.isdir(src):
            shutil.copytree(src, work / name)
            picked += 1
        elif os.path.isfile(src):
            shutil.copy(src, work / name)
            picked += 1
    client_test = os.path.join(SRC, "connector", "test_ipc_client.py")
    if os.path.isfile(client_test):
        (work / "connector").mkdir()
        shutil.copy(client_test, work / "connector" / "test_ipc_client.py")
        (work / "connector" / "__init__.py").write_text("")
    if picked == 0:
        pytest.skip("the reference test tree is empty")
    (work / "conftest.py").write_text(CONFTEST.format(root=ROOT))
    proc = subprocess.run([sys.executable, "-m", "pytest", "-q", "--no-header", "-p", "no:cacheprovider", str(work)],
                          capture_output=True, text=True, timeout=600, cwd=str(work))
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert " passed" in proc.stdout and "failed" not in proc.stdout.splitlines()[-1], tail
