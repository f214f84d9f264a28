"""Communicator set-up without a GPU: the rendezvous file and the time limits.

kutacc_comm_init replaces the reference's KUPL/MPI start-up (src/comm/kupl.cpp:50-68). These tests cover what
happens when a peer never arrives: the poll for rank 0's rendezvous record runs out, a record left by an
earlier job (or one that is not this user's regular file) is refused, and a communicator whose set-up never
completes is aborted after the host time limit. NCCL itself is replaced by a stand-in (tests/fake_nccl.c)
that has no transport, so nothing here touches a GPU. Each case runs in a child process: the library's error
flag and rank globals are process-wide.
"""
import os
import struct
import subprocess
import sys
import textwrap
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory, kutacc_lib):
    d = tmp_path_factory.mktemp("fake_nccl")
    so = str(d / "libfake_nccl.so")
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-O1", "-o", so, os.path.join(ROOT, "tests", "fake_nccl.c")])
    return so


def run_child(body, env_extra, timeout=60):
    code = "\n".join([
        "import sys, time",
        f"sys.path.insert(0, {ROOT!r})",
        "from kutacc_b200 import api",
        "api.lib()",
        "t0 = time.time()",
        "try:",
        textwrap.indent(textwrap.dedent(body).strip(), "    "),
        "    print('RESULT no error')",
        "except api.KutaccError as exc:",
        "    print('RESULT error after %.2f s:' % (time.time() - t0), str(exc).replace(chr(10), ' '))",
    ])
    env = dict(os.environ)
    env.update(env_extra)
    p = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=timeout)
    assert p.returncode == 0, p.stdout + p.stderr
    line = [ln for ln in p.stdout.splitlines() if ln.startswith("RESULT")]
    assert line, p.stdout + p.stderr
    return line[-1]


def test_rank_that_waits_alone_times_out(fake_nccl, tmp_path):
    """Rank 1 of 2 with no rank 0: the poll for the rendezvous record ends after the time limit, the call
    returns with the error flag set, and the process is still usable."""
    env = {"KUTACC_NCCL_LIB": fake_nccl, "KUTACC_RENDEZVOUS": str(tmp_path / "never_written.ncclid"),
           "KUTACC_RENDEZVOUS_TIMEOUT_S": "1"}
    res = run_child("api.comm_init(2, 1, 0)", env)
    assert "no fresh rendezvous record" in res and "rank 1" in res, res


def test_stale_or_foreign_record_is_refused(fake_nccl, tmp_path):
    path = tmp_path / "stale.ncclid"
    # (a) a record of the right shape whose stamp is older than the slack: left by an earlier job
    path.write_bytes(b"\x11" * 128 + struct.pack("<qq", int(time.time()) - 1000, 2))
    os.chmod(path, 0o600)
    env = {"KUTACC_NCCL_LIB": fake_nccl, "KUTACC_RENDEZVOUS": str(path), "KUTACC_RENDEZVOUS_TIMEOUT_S": "1",
           "KUTACC_RENDEZVOUS_SLACK_S": "5"}
    assert "no fresh rendezvous record" in run_child("api.comm_init(2, 1, 0)", env)
    # (b) a fresh record for another world size
    path.write_bytes(b"\x11" * 128 + struct.pack("<qq", int(time.time()), 4))
    assert "no fresh rendezvous record" in run_child("api.comm_init(2, 1, 0)", env)
    # (c) a fresh record that others may write to is not trusted
    path.write_bytes(b"\x11" * 128 + struct.pack("<qq", int(time.time()), 2))
    os.chmod(path, 0o666)
    assert "no fresh rendezvous record" in run_child("api.comm_init(2, 1, 0)", env)
    # (d) a symbolic link in place of the file is not followed
    real = tmp_path / "real.bin"
    real.write_bytes(b"\x11" * 128 + struct.pack("<qq", int(time.time()), 2))
    os.chmod(real, 0o600)
    link = tmp_path / "link.ncclid"
    os.symlink(real, link)
    env_link = dict(env, KUTACC_RENDEZVOUS=str(link))
    assert "no fresh rendezvous record" in run_child("api.comm_init(2, 1, 0)", env_link)


def test_fresh_record_is_accepted_then_setup_times_out(fake_nccl, tmp_path):
    """A fresh record of this user is taken; the communicator set-up that follows never completes (the stand-in
    has no peers), so the host time limit aborts it and the error names that."""
    path = tmp_path / "fresh.ncclid"
    path.write_bytes(b"\x11" * 128 + struct.pack("<qq", int(time.time()), 2))
    os.chmod(path, 0o600)
    log = tmp_path / "calls.log"
    env = {"KUTACC_NCCL_LIB": fake_nccl, "KUTACC_RENDEZVOUS": str(path), "KUTACC_RENDEZVOUS_TIMEOUT_S": "5",
           "KUTACC_COMM_TIMEOUT_S": "1", "FAKE_NCCL_LOG": str(log)}
    res = run_child("api.comm_init(2, 1, 0)", env)
    assert "ran out of time and was aborted" in res, res
    calls = log.read_text().split()
    assert calls == ["ncclCommInitRankConfig", "ncclCommAbort"], calls


def test_setup_with_given_id_times_out_and_rank0_publishes_private_file(fake_nccl, tmp_path):
    log = tmp_path / "calls.log"
    env = {"KUTACC_NCCL_LIB": fake_nccl, "KUTACC_COMM_TIMEOUT_S": "1", "FAKE_NCCL_LOG": str(log)}
    res = run_child("api.comm_init(2, 0, 0, api.comm_unique_id())", env)
    assert "ran out of time and was aborted" in res, res
    assert log.read_text().split() == ["ncclGetUniqueId", "ncclCommInitRankConfig", "ncclCommAbort"]
    # rank 0 through the file: the record it publishes is a private regular file of this user
    path = tmp_path / "pub.ncclid"
    env = {"KUTACC_NCCL_LIB": fake_nccl, "KUTACC_RENDEZVOUS": str(path), "KUTACC_COMM_TIMEOUT_S": "1"}
    res = run_child("api.comm_init(2, 0, 0)", env)
    assert "ran out of time and was aborted" in res, res
    st = os.stat(path)
    assert st.st_uid == os.getuid() and (st.st_mode & 0o077) == 0 and st.st_size == 144
    world = struct.unpack("<qq", path.read_bytes()[128:])[1]
    assert world == 2
