"""Parameter server on the CPU: record format, put/get/update semantics, loopback clients, sharding."""
import struct

import numpy as np
import pytest
import torch


def test_record_format_layout_and_roundtrip():
    from recstore_b200.ps import pack_records, unpack_records
    keys = torch.tensor([7, 1 << 40, 3])
    vals = torch.arange(12, dtype=torch.float32).view(3, 4)
    buf = pack_records(keys, vals, dims=[4, 0, 4])            # middle record "missing"
    n, = struct.unpack_from("<i", buf, 0)
    ends = struct.unpack_from("<3i", buf, 4)
    assert n == 3 and ends == (16 + 12 + 16, 16 + 28 + 12, 16 + 28 + 12 + 28) and len(buf) == ends[-1]
    k0, d0 = struct.unpack_from("<Qi", buf, 16)
    assert (k0, d0) == (7, 4) and struct.unpack_from("<4f", buf, 28) == (0.0, 1.0, 2.0, 3.0)
    k, d, v = unpack_records(buf, 4)
    assert k.tolist() == keys.tolist() and d.tolist() == [4, 0, 4]
    assert torch.equal(v[0], vals[0]) and v[1].abs().sum() == 0 and torch.equal(v[2], vals[2])
    with pytest.raises(Exception):
        unpack_records(buf[:20], 4)


@pytest.mark.parametrize("engine", ["KVEngineMap", "KVEngineChunkHash"])
def test_ps_client_server_mirror(engine, tmp_path):
    """clear -> get(empty) -> put -> get(equal) -> update -> checkpoint -> clear -> get(empty) -> load, plus the
    10-round random put/get mirror of the reference's python client test."""
    from recstore_b200.ps import ParameterServer, ParameterClient
    dim = 8
    srv = ParameterServer(engine, {"dim": dim, "capacity": 100000, "optimizer": "rowwise_adagrad", "lr": 0.1, "eps": 1e-10})
    port = srv.serve(0)
    cli = ParameterClient("127.0.0.1", port, 0, dim)
    cli.ClearPS()
    keys = torch.arange(5000)
    out, found = cli.GetParameterWithMask(keys)
    assert not found.any() and out.abs().sum() == 0                     # missing key -> zero row, no error
    rng = np.random.default_rng(0)
    mirror = torch.zeros(20000, dim)
    present = torch.zeros(20000, dtype=torch.bool)
    for _ in range(10):
        k = torch.from_numpy(rng.choice(20000, size=4500, replace=False))   # > 2 sub-requests of 2000 keys
        v = torch.from_numpy(rng.standard_normal((4500, dim)).astype(np.float32))
        cli.PutParameter(k, v)
        mirror[k] = v; present[k] = True
        q = torch.from_numpy(rng.integers(0, 20000, size=5000))
        got = cli.GetParameter(q)
        assert torch.equal(got, mirror[q] * present[q].unsqueeze(1))
    # gradient verb with duplicates: row-wise Adagrad, post-step state for every occurrence
    k = torch.tensor([5, 5, 9])
    cli.PutParameter(torch.tensor([5, 9]), torch.ones(2, dim))
    g = torch.tensor([[1.0] * dim, [3.0] * dim, [2.0] * dim])
    assert cli.UpdateParameter(k, g) == 3
    s5, s9 = 1.0 + 9.0, 4.0
    exp5 = 1 - 0.1 * (1 + 3) / (s5 ** 0.5 + 1e-10)
    exp9 = 1 - 0.1 * 2 / (s9 ** 0.5 + 1e-10)
    got = cli.GetParameter(torch.tensor([5, 9]))
    assert torch.allclose(got[0], torch.full((dim,), exp5), atol=1e-6) and torch.allclose(got[1], torch.full((dim,), exp9), atol=1e-6)
    mirror[5] = got[0]; mirror[9] = got[1]; present[5] = True; present[9] = True
    # async window
    rid = cli.GetParameterAsync(torch.arange(3000))
    cli.WaitRPCFinish(rid)
    assert cli.QueryRPCFinished(rid)
    assert torch.equal(cli.GetReceiveBuffer(rid), (mirror * present.unsqueeze(1))[:3000])
    cli.RevokeRPCResource(rid)
    # asynchronous put: the caller's buffer may be reused at once, the rows land when the rpc has finished
    buf = torch.full((3, dim), 7.0)
    rid = cli.FakePutParameter(torch.tensor([11, 12, 13]), buf)
    buf.zero_()
    cli.WaitRPCFinish(rid)
    assert cli.QueryRPCFinished(rid) and torch.equal(cli.GetParameter(torch.tensor([11, 12, 13])), torch.full((3, dim), 7.0))
    cli.RevokeRPCResource(rid)
    mirror[11:14] = 7.0; present[11:14] = True
    # checkpoint round trip through the server
    ck = str(tmp_path / "ps.ckpt")
    cli.SaveCkpt(ck)
    n_before = cli.Stats()["keys_stored"]
    cli.ClearPS()
    assert cli.Stats()["keys_stored"] == 0 and cli.GetParameter(torch.tensor([5])).abs().sum() == 0
    cli.LoadCkpt(None, [ck])
    assert cli.Stats()["keys_stored"] == n_before
    assert torch.equal(cli.GetParameter(torch.arange(20000)), mirror * present.unsqueeze(1))
    # the optimizer state came back too: one more update continues from s5
    cli.UpdateParameter(torch.tensor([5]), torch.full((1, dim), 2.0))
    assert torch.allclose(cli.GetParameter(torch.tensor([5]))[0], torch.full((dim,), exp5 - 0.1 * 2 / ((s5 + 4) ** 0.5)), atol=1e-6)
    with pytest.raises(Exception):
        cli.LoadCkpt(None, [str(tmp_path / "missing.ckpt")])
    cli.LoadFakeData(100)
    assert torch.equal(cli.GetParameter(torch.tensor([42]))[0], torch.full((dim,), 42.0))
    cli.close(); srv.close()


def test_all_shards_client():
    from recstore_b200.ps import ParameterServer, ParameterClient, AllShardsParameterClient, ShardManager
    dim = 4
    servers = [ParameterServer("KVEngineExtendibleHash", {"dim": dim, "capacity": 50000, "optimizer": "sgd", "lr": 1.0}) for _ in range(2)]
    clients = [ParameterClient("127.0.0.1", s.serve(0), i, dim) for i, s in enumerate(servers)]
    allc = AllShardsParameterClient(clients)
    keys = torch.arange(10000)
    vals = keys.float().unsqueeze(1).repeat(1, dim)
    allc.PutParameter(keys, vals)
    owner = ShardManager.KeyPartition(keys, 2)
    assert len(servers[0]) == int((owner == 0).sum()) and len(servers[1]) == int((owner == 1).sum())
    assert abs(len(servers[0]) - 5000) < 400                           # the hash spreads keys
    perm = torch.randperm(10000)
    assert torch.equal(allc.GetParameter(perm), vals[perm])
    assert allc.UpdateParameter(torch.tensor([1, 2, 3]), torch.ones(3, dim)) == 3
    assert torch.equal(allc.GetParameter(torch.tensor([1, 2, 3])), vals[1:4] - 1)
    for c in clients:
        c.close()
    for s in servers:
        s.close()


def test_client_connect_failure_is_an_error():
    from recstore_b200.ps import ParameterClient
    from recstore_b200 import _lib
    with pytest.raises(_lib.RecStoreError):
        ParameterClient("127.0.0.1", 1, 0, 4)


def test_record_parser_survives_random_and_truncated_buffers():
    """Property test of the wire parser: every well-formed buffer round-trips; truncations, bit flips in the header and
    random bytes are either parsed consistently or rejected with an error - never a crash or an out-of-bounds read
    (the test runs in-process, so a wild read would take the interpreter down)."""
    from hypothesis import given, settings, strategies as st
    from recstore_b200 import _lib
    from recstore_b200.ps import pack_records, unpack_records

    @settings(max_examples=120, deadline=None)
    @given(st.integers(0, 12), st.integers(1, 9), st.data())
    def run(n, dim, data):
        keys = torch.tensor(data.draw(st.lists(st.integers(0, (1 << 62)), min_size=n, max_size=n)), dtype=torch.int64)
        vals = torch.arange(n * dim, dtype=torch.float32).view(n, dim) * 0.5
        present = data.draw(st.lists(st.booleans(), min_size=n, max_size=n))
        buf = pack_records(keys, vals, dims=[dim if p else 0 for p in present])
        k, d, v = unpack_records(buf, dim)
        assert k.tolist() == keys.tolist() and d.tolist() == [dim if p else 0 for p in present]
        for i, p in enumerate(present):
            assert torch.equal(v[i], vals[i]) if p else float(v[i].abs().sum()) == 0.0
        cut = data.draw(st.integers(0, max(0, len(buf) - 1)))
        mangled = bytearray(buf[:cut]) if data.draw(st.booleans()) else bytearray(buf)
        for _ in range(data.draw(st.integers(0, 3))):
            if mangled:
                pos = data.draw(st.integers(0, min(len(mangled), 4 + 4 * n + 12) - 1))
                mangled[pos] ^= 1 << data.draw(st.integers(0, 7))
        try:
            k2, d2, v2 = unpack_records(bytes(mangled), dim)
            assert k2.numel() == d2.numel() == v2.shape[0]
        except _lib.RecStoreError:
            pass
        junk = data.draw(st.binary(min_size=0, max_size=64))
        try:
            unpack_records(junk, dim)
        except _lib.RecStoreError:
            pass

    run()


def test_server_survives_malformed_frames():
    """Hostile or broken clients: wrong magic, absurd lengths, truncated payloads, unknown verbs, key counts that do not
    divide, record buffers with wild offsets.  The connection concerned is dropped; the server keeps serving others."""
    import random
    import socket
    from recstore_b200.ps import ParameterClient, ParameterServer
    srv = ParameterServer("KVEngineMap", {"capacity": 4096, "dim": 4})
    port = srv.serve(0)
    good = ParameterClient("127.0.0.1", port, 0, 4)
    good.PutParameter(torch.tensor([1, 2, 3]), torch.arange(12, dtype=torch.float32).view(3, 4))
    MAGIC = 0x52535053
    rnd = random.Random(0)

    def send(raw: bytes):
        s = socket.create_connection(("127.0.0.1", port), timeout=5)
        try:
            s.sendall(raw)
            s.settimeout(0.3)
            try:
                s.recv(64)
            except (socket.timeout, ConnectionError):
                pass
        finally:
            s.close()

    frames = [
        struct.pack("<IIQ", 0xDEADBEEF, 1, 8) + b"\x00" * 8,                        # wrong magic
        struct.pack("<IIQ", MAGIC, 1, 1 << 40),                                     # absurd length
        struct.pack("<IIQ", MAGIC, 1, (256 << 20) + 8),                             # just over the frame limit
        struct.pack("<IIQ", MAGIC, 1, 64) + b"\x01" * 10,                           # truncated payload
        struct.pack("<IIQ", MAGIC, 1, 12) + b"\x01" * 12,                           # GET whose length is not a multiple of 8
        struct.pack("<IIQ", MAGIC, 77, 0),                                          # unknown verb
        struct.pack("<IIQ", MAGIC, 2, 8) + struct.pack("<ii", 1 << 30, 0),          # PUT announcing 2^30 records
        struct.pack("<IIQ", MAGIC, 3, 24) + struct.pack("<iiQi", 1, 1 << 28, 5, 4), # UPDATE with an end offset far outside
        struct.pack("<IIQ", MAGIC, 2, 20) + struct.pack("<iiQi", 1, -5, 5, 4),      # negative offset
        b"\x00" * 3,                                                                # less than a header
    ]
    for _ in range(40):
        op, ln = rnd.randrange(0, 12), rnd.randrange(0, 200)
        body = bytes(rnd.randrange(256) for _ in range(rnd.randrange(0, ln + 1)))
        frames.append(struct.pack("<IIQ", MAGIC if rnd.random() < 0.8 else rnd.getrandbits(32), op if op not in (4, 5, 6, 7) else 1, ln) + body)
    for fr in frames:
        send(fr)
        got = good.GetParameter(torch.tensor([2, 3, 99]))
        assert got[0].tolist() == [4.0, 5.0, 6.0, 7.0] and got[1].tolist() == [8.0, 9.0, 10.0, 11.0] and float(got[2].abs().sum()) == 0.0
    assert good.Stats()["keys_stored"] >= 3
    good.close()
    srv.close()


def test_checkpoint_loader_rejects_corrupt_files(tmp_path):
    """Truncated or bit-flipped PS checkpoints give an error (or load the intact prefix consistently); they never take
    the process down."""
    import random
    from recstore_b200 import _lib
    from recstore_b200.ps import ParameterServer
    ps = ParameterServer("KVEngineMap", {"capacity": 4096, "dim": 4})
    ps.PutParameter(torch.arange(100), torch.rand(100, 4))
    good = str(tmp_path / "c.bin")
    ps.SaveCkpt(good)
    raw = open(good, "rb").read()
    rnd = random.Random(0)
    errors = 0
    for _ in range(150):
        b = bytearray(raw[:rnd.randrange(0, len(raw))]) if rnd.random() < 0.5 else bytearray(raw)
        for _ in range(rnd.randrange(0, 4)):
            if b:
                b[rnd.randrange(0, min(len(b), 64))] ^= 1 << rnd.randrange(8)
        bad = str(tmp_path / "m.bin")
        open(bad, "wb").write(bytes(b))
        ps2 = ParameterServer("KVEngineMap", {"capacity": 4096, "dim": 4})
        try:
            ps2.LoadCkpt(bad)
        except _lib.RecStoreError:
            errors += 1
        ps2.close()
    assert errors > 50
    ps3 = ParameterServer("KVEngineMap", {"capacity": 4096, "dim": 4})
    ps3.LoadCkpt(good)
    assert len(ps3) == 100 and torch.equal(ps3.GetParameter(torch.arange(100)), ps.GetParameter(torch.arange(100)))
    with pytest.raises(_lib.RecStoreError):
        ps3.LoadCkpt(str(tmp_path / "missing.bin"))


def test_grpc_transport_mirror_commands_and_wire_format(tmp_path):
    """The parameter service over gRPC (the reference's transport, src/grpc_ps/proto/ps.proto): put / get / update
    against a Python mirror over several sub-requests, the three commands, checkpoints, absent keys as zero rows with a
    cleared mask, the asynchronous form, the sharded fan-out, and the raw wire layout of a request."""
    import struct
    import grpc
    from recstore_b200.ps.client import AllShardsParameterClient, ParameterServer, unpack_records
    from recstore_b200.ps import grpc_transport as gt
    D = 16
    ps = ParameterServer("KVEngineMap", {"dim": D, "capacity": 1 << 16, "optimizer": "sgd", "lr": 0.5})
    srv = gt.GrpcParameterServer(ps)
    cli = gt.GrpcParameterClient("127.0.0.1", srv.port, 0, D)
    g = torch.Generator().manual_seed(0)
    keys = torch.randperm(50000, generator=g)[:5000]                  # 3 sub-requests of MAX_PARAMETER_BATCH keys
    vals = torch.randn(5000, D, generator=g)
    assert cli.PutParameter(keys, vals)
    assert torch.equal(cli.GetParameter(keys), vals) and len(ps) == 5000
    q = torch.cat([keys[:10], torch.tensor([60001, 60002])])
    rows, found = cli.GetParameterWithMask(q)
    assert found.tolist() == [True] * 10 + [False] * 2 and rows[10:].abs().sum() == 0 and torch.equal(rows[:10], vals[:10])
    grads = torch.ones(100, D)
    assert cli.UpdateParameter(keys[:100], grads) == 100
    assert torch.allclose(cli.GetParameter(keys[:100]), vals[:100] - 0.5)
    rid = cli.GetParameterAsync(keys[200:2700])
    cli.WaitRPCFinish(rid)
    assert cli.QueryRPCFinished(rid) and torch.equal(cli.GetReceiveBuffer(rid), vals[200:2700])
    cli.RevokeRPCResource(rid)
    ck = str(tmp_path / "ps.ckpt")
    assert cli.SaveCkpt(ck) and cli.ClearPS() and len(ps) == 0
    assert cli.LoadCkpt(emb_file_path=[ck]) and len(ps) == 5000 and torch.equal(cli.GetParameter(keys[100:300]), vals[100:300])
    assert cli.ClearPS() and cli.LoadFakeData(300)
    assert torch.equal(cli.GetParameter(torch.arange(300))[:, 0], torch.arange(300).float())
    st = cli.Stats()
    assert st["keys_stored"] == 300 and st["requests"] > 10
    assert cli.HealthCheck() and cli.HealthCheck("xmhps.ParameterService")
    with pytest.raises(grpc.RpcError) as he:
        cli.HealthCheck("no.such.Service")
    assert he.value.code() == grpc.StatusCode.NOT_FOUND
    # server reflection: the services are listed, the service's symbol resolves to a descriptor that names its methods
    assert set(cli.ListServices()) >= {"xmhps.ParameterService", "grpc.health.v1.Health", "grpc.reflection.v1alpha.ServerReflection"}
    from google.protobuf import descriptor_pb2
    rep = cli.Reflect(file_containing_symbol="xmhps.ParameterService", host="h")
    assert rep.valid_host == "h" and rep.original_request.file_containing_symbol == "xmhps.ParameterService"
    fd = descriptor_pb2.FileDescriptorProto.FromString(rep.file_descriptor_response.file_descriptor_proto[0])
    assert fd.package == "xmhps" and [m.name for m in fd.service[0].method] == ["GetParameter", "Command", "PutParameter", "UpdateParameter"]
    assert {m.name for m in fd.message_type} >= {"GetParameterRequest", "PutParameterResponse"}
    assert cli.Reflect(file_by_filename=fd.name).file_descriptor_response.file_descriptor_proto[0] == fd.SerializeToString()
    assert cli.Reflect(file_containing_symbol="xmhps.GetParameterRequest").WhichOneof("message_response") == "file_descriptor_response"
    miss = cli.Reflect(file_containing_symbol="no.such.Symbol")
    assert miss.WhichOneof("message_response") == "error_response" and miss.error_response.error_code == grpc.StatusCode.NOT_FOUND.value[0]
    assert cli.Reflect().error_response.error_code == grpc.StatusCode.INVALID_ARGUMENT.value[0]
    v1 = cli._channel.stream_stream("/grpc.reflection.v1.ServerReflection/ServerReflectionInfo",
                                    request_serializer=gt.ServerReflectionRequest.SerializeToString,
                                    response_deserializer=gt.ServerReflectionResponse.FromString)
    assert len(next(iter(v1(iter([gt.ServerReflectionRequest(list_services="")]), timeout=10))).list_services_response.service) == 4
    # the bytes on the wire: field 1 = raw little-endian u64 keys; the answer is one packed record block
    raw = cli._channel.unary_unary("/xmhps.ParameterService/GetParameter")(
        b"\x0a\x10" + struct.pack("<2Q", 7, 999999), timeout=10)
    assert raw[0] == 0x0a                                                   # GetParameterResponse.parameter_value
    blob = gt.GetParameterResponse.FromString(raw).parameter_value
    k, d, v = unpack_records(blob, D)
    assert k.tolist() == [7, 999999] and d.tolist() == [D, 0] and v[0, 0] == 7.0
    # malformed requests are refused, the server keeps serving
    with pytest.raises(grpc.RpcError) as e:
        cli._get(gt.GetParameterRequest(keys=b"12345"), timeout=10)
    assert e.value.code() == grpc.StatusCode.INVALID_ARGUMENT
    with pytest.raises(grpc.RpcError):
        cli._put(gt.PutParameterRequest(parameter_value=b"\xff\xff\xff\x7f" + b"junk"), timeout=10)
    with pytest.raises(grpc.RpcError):
        cli.LoadCkpt(emb_file_path=str(tmp_path / "missing.ckpt"))
    assert cli.GetParameter([5])[0, 0] == 5.0
    # two shards behind the fan-out client
    ps2 = ParameterServer("KVEngineChunkHash", {"dim": D, "capacity": 1 << 16})
    srv2 = gt.GrpcParameterServer(ps2)
    both = AllShardsParameterClient([cli, gt.GrpcParameterClient("127.0.0.1", srv2.port, 1, D)])
    both.ClearPS()
    both.PutParameter(keys, vals)
    assert torch.equal(both.GetParameter(keys), vals) and len(ps) + len(ps2) == 5000 and min(len(ps), len(ps2)) > 2000
    # a server that is gone is an error within the timeout, not a hang
    srv2.stop(0)
    dead = gt.GrpcParameterClient("127.0.0.1", srv2.port, 1, D, timeout_s=1.0)
    with pytest.raises(grpc.RpcError):
        dead.GetParameter([1, 2, 3])
    srv.stop(0)


def test_task_providers_fifo_and_priority_levels():
    """FIFO order; the priority provider draws level i with probability ~ i x queue length, raises a class on
    ImprovePriority, keeps levels relative (nobody left at level 1 -> everybody moves down) and caps at `levels`."""
    from recstore_b200.ps.client import TaskProvider
    f = TaskProvider("fifo")
    for i in range(10):
        f.PutTask(i, i % 3)
    assert f.LeftTask() == 10 and [f.GetTask() for _ in range(10)] == list(range(10)) and f.GetTask() is None and not f.ExistTask()
    p = TaskProvider("priority", levels=4, seed=7)
    assert p.LevelOf(1) == 1
    p.PutTask(0, 1); p.PutTask(0, 2)                      # both classes known at level 1
    p.ImprovePriority(2); p.ImprovePriority(2)
    assert (p.LevelOf(1), p.LevelOf(2)) == (1, 3)
    for _ in range(5):
        p.ImprovePriority(2)
    assert p.LevelOf(2) == 4                              # capped
    p.ImprovePriority(1)                                  # 1 -> 2: nobody at level 1 any more, so (2, 4) -> (1, 3)
    assert (p.LevelOf(1), p.LevelOf(2)) == (1, 3)
    while p.GetTask() is not None:
        pass
    # equal backlogs of class 1 (level 1, ids < 1000) and class 2 (level 3, ids >= 1000): the first draws favour class 2 by 3:1
    for i in range(600):
        p.PutTask(i, 1); p.PutTask(1000 + i, 2)
    first = [p.GetTask() for _ in range(200)]
    hi = sum(1 for t in first if t >= 1000)
    assert 125 <= hi <= 175, hi                           # expectation 150, sigma ~ 6
    lo_ids = [t for t in first if t < 1000]
    assert lo_ids == sorted(lo_ids)                       # FIFO inside a level
    rest = []
    while p.ExistTask():
        rest.append(p.GetTask())
    assert sorted(first + rest) == sorted(list(range(600)) + list(range(1000, 1600)))   # nothing lost, nothing starved


@pytest.mark.parametrize("scheduler", ["fifo", "priority"])
def test_pooled_server_keeps_request_order_per_connection(scheduler):
    """Front-end threads + worker pool: pipelined sub-requests of several concurrent clients come back in order (the
    client checks every key of every answer), updates from all clients add up, and the priority verb answers."""
    import threading
    from recstore_b200.ps.client import ParameterClient, ParameterServer
    D = 8
    ps = ParameterServer("KVEngineMap", {"dim": D, "capacity": 1 << 17, "optimizer": "sgd", "lr": 1.0})
    port = ps.serve(0, workers=4, scheduler=scheduler)
    ps.LoadFakeData(60000)
    errs = []
    known = threading.Barrier(4)

    def client(seed):
        try:
            c = ParameterClient("127.0.0.1", port, 0, D)
            c.GetParameter([seed])                     # the server knows this connection's class from its first task on
            known.wait(30)
            if seed == 0:                              # levels are relative: somebody else has to be at level 1
                assert c.ImprovePriority() == (2 if scheduler == "priority" else 1)
            g = torch.Generator().manual_seed(seed)
            for _ in range(6):
                k = torch.randint(0, 50000, (9000,), generator=g)          # 5 pipelined sub-requests
                rows, found = c.GetParameterWithMask(k)
                assert bool(found.all()) and torch.equal(rows[:, 0], k.float())
            c.UpdateParameter(torch.arange(50000, 50100), torch.ones(100, D))
            c.close()
        except BaseException as e:      # noqa: BLE001
            errs.append(repr(e))
    ts = [threading.Thread(target=client, args=(i,)) for i in range(4)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errs, errs
    c = ParameterClient("127.0.0.1", port, 0, D)
    base = torch.arange(50000, 50100).float().unsqueeze(1).repeat(1, D)
    assert torch.equal(c.GetParameter(torch.arange(50000, 50100)), base - 4.0)
    st = c.Stats()
    assert st["pooled_requests"] >= 4 * (6 * 5 + 1) and st["requests"] > st["pooled_requests"]
    c.close()
    ps.close()


def test_grpc_server_survives_random_request_bytes():
    """Every method fed with random and truncated byte strings: the call ends with a gRPC status (or a well-formed answer
    when the bytes happen to parse), never with a dead server; afterwards the shard still answers and still holds its rows."""
    import random
    import grpc
    from recstore_b200.ps.client import ParameterServer
    from recstore_b200.ps import grpc_transport as gt
    D = 8
    ps = ParameterServer("KVEngineMap", {"dim": D, "capacity": 1 << 14})
    ps.LoadFakeData(500)
    srv = gt.GrpcParameterServer(ps)
    cli = gt.GrpcParameterClient("127.0.0.1", srv.port, 0, D, timeout_s=5.0)
    good_put = gt.PutParameterRequest(parameter_value=__import__("recstore_b200.ps.client", fromlist=["pack_records"]).pack_records(
        torch.arange(4), torch.ones(4, D))).SerializeToString()
    rng = random.Random(7)
    outcomes = {"ok": 0, "status": 0}
    for method in ("GetParameter", "PutParameter", "UpdateParameter", "Command"):
        call = cli._channel.unary_unary(f"/xmhps.ParameterService/{method}")
        for trial in range(40):
            if trial % 4 == 0:
                blob = good_put[: rng.randrange(len(good_put))]                  # a truncated valid message
            elif trial % 4 == 1:
                b = bytearray(good_put)
                b[rng.randrange(len(b))] ^= 1 << rng.randrange(8)                  # one flipped bit
                blob = bytes(b)
            else:
                blob = bytes(rng.randrange(256) for _ in range(rng.randrange(1, 200)))
            try:
                call(blob, timeout=5)
                outcomes["ok"] += 1
            except grpc.RpcError as e:
                assert e.code() in (grpc.StatusCode.INVALID_ARGUMENT, grpc.StatusCode.INTERNAL, grpc.StatusCode.NOT_FOUND,
                                    grpc.StatusCode.FAILED_PRECONDITION, grpc.StatusCode.UNKNOWN), e.code()
                outcomes["status"] += 1
    assert outcomes["status"] > 20, outcomes
    assert cli.HealthCheck()
    got = cli.GetParameter(torch.arange(100, 110))
    assert got.shape == (10, D)
    srv.stop(0)


def test_server_throughput_monitor_reports_traffic_per_period(capfd):
    """The server's monitor thread (role of the MB/s line of src/grpc_ps/grpc_ps_server_async.cpp:109-117)."""
    import time
    from recstore_b200.ps import ParameterClient, ParameterServer
    D = 8
    srv = ParameterServer("KVEngineMap", {"dim": D, "capacity": 10000})
    port = srv.serve(0)
    srv.start_monitor(0.1)
    srv.start_monitor(0.1)                                   # a second start is a no-op
    cli = ParameterClient("127.0.0.1", port, 0, D)
    cli.LoadFakeData(5000)
    t0, best = time.time(), 0.0
    while time.time() - t0 < 0.6:
        cli.GetParameter(torch.arange(2000))
        best = max(best, srv.monitor_last()["mkeys_per_s"])
    m = srv.monitor_last()
    assert m["periods"] >= 2 and best > 0.01 and m["mb_per_s"] == pytest.approx(m["mkeys_per_s"] * (12 + 4 * D), rel=1e-6)
    time.sleep(0.35)                                          # idle periods read zero and print nothing
    assert srv.monitor_last()["mkeys_per_s"] == 0.0
    srv.stop_monitor()
    n = srv.monitor_last()["periods"]
    time.sleep(0.25)
    assert srv.monitor_last()["periods"] == n
    cli.close()
    srv.close()                                               # closing with or without a running monitor is fine
    err = capfd.readouterr().err
    lines = [l for l in err.splitlines() if l.startswith("PS throughput:")]
    assert len(lines) >= 2 and "Mkeys/s" in lines[0] and "MB/s" in lines[0]      # one line per period that saw traffic


def test_client_benchmark_thread_cut_off_reports_every_thread_count():
    """One run, the whole load curve: sender threads are stopped a few at a time
    (src/benchmark/benchmark_client_common.h:156-184 `thread_cut_off`)."""
    from recstore_b200.bench.ps_client import closed_loop
    from recstore_b200.ps import ParameterServer
    srv = ParameterServer("KVEngineMap", {"dim": 8, "capacity": 20000})
    srv.LoadFakeData(10000)
    port = srv.serve(0)
    out = closed_loop("127.0.0.1", port, 8, threads=5, window=2, batch=100, alpha=0.9, key_space=10000, seconds=999, quiet=True,
                      cut_off_period=0.15, cut_off_stride=2)
    assert out["mode"] == "closed_cut_off" and [c["threads"] for c in out["by_threads"]] == [5, 3, 1]
    assert all(c["keys_per_s"] > 0 for c in out["by_threads"]) and out["seconds"] < 60
    srv.close()


def test_server_listens_on_the_address_it_is_given():
    """Loopback by default; any IPv4 address on request (the reference's server listens on 0.0.0.0)."""
    from recstore_b200.ps import ParameterClient, ParameterServer
    srv = ParameterServer("KVEngineMap", {"dim": 4, "capacity": 1000})
    port = srv.serve(0, host="0.0.0.0", workers=2)
    cli = ParameterClient("127.0.0.1", port, 0, 4)
    cli.PutParameter(torch.tensor([3]), torch.ones(1, 4))
    assert torch.equal(cli.GetParameter(torch.tensor([3])), torch.ones(1, 4)) and cli.Stats()["pooled_requests"] >= 2
    cli.close()
    srv.close()
    bad = ParameterServer("KVEngineMap", {"dim": 4, "capacity": 1000})
    with pytest.raises(Exception, match="not an IPv4 address"):
        bad.serve(0, host="not-an-address")
    with pytest.raises(Exception, match="cannot listen"):
        bad.serve(0, host="203.0.113.7")                      # a documentation address: not on this machine
    assert bad.serve(0) > 0                                   # the shard is still usable
    bad.close()


@pytest.mark.parametrize("transport", ["tcp", "grpc"])
def test_stand_alone_server_process_serves_until_sigterm_and_saves(tmp_path, transport):
    """`python -m recstore_b200.ps.server`: a shard as a process of its own (the reference's grpc_ps_server binary):
    ready line, warm-up of its partition, requests from a client, SIGTERM -> checkpoint -> a second server restores it."""
    import os, re, signal, subprocess, sys, time
    from recstore_b200.ps import ParameterClient
    from recstore_b200.ps.client import ShardManager
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ck = str(tmp_path / "shard.ckpt")

    def start(*extra):
        import queue, threading
        p = subprocess.Popen([sys.executable, "-m", "recstore_b200.ps.server", "--port", "0", "--dim", "8", "--capacity", "20000",
                              "--transport", transport, "--workers", "2", *extra],
                             stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=root)
        q = queue.Queue()
        threading.Thread(target=lambda: [q.put(l) for l in iter(p.stdout.readline, "")], daemon=True).start()
        lines, t0 = [], time.time()
        while time.time() - t0 < 120 and p.poll() is None:
            try:
                line = q.get(timeout=0.5)
            except queue.Empty:
                continue
            lines.append(line)
            m = re.search(r"listening on [0-9.]+:([0-9]+)", line)
            if m:
                p._lines = q                               # what it prints later is read from here
                return p, int(m.group(1)), lines
        p.kill()
        raise AssertionError("the server never got ready: " + "".join(lines))

    def client(port):
        if transport == "grpc":
            from recstore_b200.ps.grpc_transport import GrpcParameterClient
            return GrpcParameterClient("127.0.0.1", port, 0, 8)
        return ParameterClient("127.0.0.1", port, 0, 8)
    p, port, lines = start("--warm", "3000", "--shard_id", "1", "--num_shards", "2", "--save_on_exit", ck)
    mine = int((ShardManager.KeyPartition(torch.arange(1, 3001), 2) == 1).sum())
    assert any(f"warmed {mine} keys of shard 1/2" in l for l in lines)
    c = client(port)
    k = torch.arange(1, 3001)
    own = ShardManager.KeyPartition(k, 2) == 1
    got = c.GetParameter(k)
    assert torch.equal(got[own][:, 0], k[own].float()) and float(got[~own].abs().sum()) == 0      # only this shard's keys are here
    c.PutParameter(torch.tensor([777777]), torch.full((1, 8), 5.0))
    c.close()
    p.send_signal(signal.SIGTERM)
    assert p.wait(timeout=60) == 0
    time.sleep(0.2)
    out = "".join(p._lines.get() for _ in range(p._lines.qsize()))
    assert '"stopped"' in out and os.path.exists(ck)
    p2, port2, _ = start("--load_ckpt", ck)
    c2 = client(port2)
    assert torch.equal(c2.GetParameter(torch.tensor([777777])), torch.full((1, 8), 5.0)) and c2.Stats()["keys_stored"] == mine + 1
    c2.close()
    p2.send_signal(signal.SIGINT)
    assert p2.wait(timeout=60) == 0


@pytest.mark.parametrize("engine", ["KVEngineChunkHash", "KVEnginePoolMap"])
def test_server_on_a_persistent_engine_restarts_with_rows_and_optimizer_state(tmp_path, engine):
    """A shard whose engine lives in files needs no checkpoint to restart: the rows are there, and so is the row-wise
    Adagrad state (the second update of a row after the restart is smaller than the first by 1 / sqrt(2))."""
    import queue, threading
    from recstore_b200.ps import ParameterClient, server
    argv = ["--port", "0", "--dim", "8", "--capacity", "5000", "--engine", engine, "--path", str(tmp_path / "shard"), "--lr", "0.01"]

    def start():
        ev, ready = threading.Event(), queue.Queue()
        t = threading.Thread(target=server.main, args=(argv, ev, ready.put))
        t.start()
        return ev, t, ParameterClient("127.0.0.1", ready.get(timeout=60), 0, 8)
    ev, t, c = start()
    c.PutParameter(torch.arange(100), torch.arange(100).float().unsqueeze(1).expand(-1, 8).contiguous())
    c.UpdateParameter(torch.tensor([5]), torch.ones(1, 8))
    v5 = c.GetParameter(torch.tensor([5]))
    assert torch.allclose(v5, torch.full((1, 8), 5.0 - 0.01), atol=1e-6)
    c.close(); ev.set(); t.join(30)
    ev, t, c = start()
    got = c.GetParameter(torch.arange(100))
    assert c.Stats()["keys_stored"] == 100 and torch.equal(got[7], torch.full((8,), 7.0)) and torch.equal(got[5:6], v5)
    c.UpdateParameter(torch.tensor([5]), torch.ones(1, 8))
    step2 = float((v5 - c.GetParameter(torch.tensor([5]))).abs().max())
    assert step2 == pytest.approx(0.01 / 2 ** 0.5, rel=1e-3)
    c.close(); ev.set(); t.join(30)
    assert not t.is_alive()


@pytest.mark.parametrize("engine", ["KVEngineChunkHash", "KVEnginePoolMap"])
def test_server_process_killed_without_warning_recovers_its_rows(tmp_path, engine):
    """Crash recovery at the level a user sees: the shard process is killed (SIGKILL: no flush, no goodbye), a new one on
    the same directory serves every row that had been acknowledged."""
    import os, queue, re, signal, subprocess, sys, threading, time
    from recstore_b200.ps import ParameterClient
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "recstore_b200.ps.server", "--port", "0", "--dim", "8", "--capacity", "20000", "--engine", engine,
           "--path", str(tmp_path / "shard")]

    def start():
        p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=root)
        q = queue.Queue()
        threading.Thread(target=lambda: [q.put(l) for l in iter(p.stdout.readline, "")], daemon=True).start()
        t0 = time.time()
        while time.time() - t0 < 120 and p.poll() is None:
            try:
                m = re.search(r"listening on [0-9.]+:([0-9]+)", q.get(timeout=0.5))
            except queue.Empty:
                continue
            if m:
                return p, int(m.group(1))
        p.kill()
        raise AssertionError("the server never got ready")
    p, port = start()
    c = ParameterClient("127.0.0.1", port, 0, 8)
    keys = torch.arange(1, 5001)
    c.PutParameter(keys, keys.float().unsqueeze(1).expand(-1, 8).contiguous())
    assert c.Stats()["keys_stored"] == 5000                  # every put above has been answered
    c.close()
    os.kill(p.pid, signal.SIGKILL)                           # this test's own child, by its pid
    assert p.wait(timeout=30) == -signal.SIGKILL
    p2, port2 = start()
    c2 = ParameterClient("127.0.0.1", port2, 0, 8)
    got, found = c2.GetParameterWithMask(keys)
    assert bool(found.all()) and torch.equal(got[:, 0], keys.float()) and torch.equal(got[:, 7], keys.float())
    c2.close()
    p2.send_signal(signal.SIGTERM)
    assert p2.wait(timeout=60) == 0
