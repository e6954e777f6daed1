"""Prototypes of the C API groups added on top of the device-communicator core
(optimizer / model kernels, CPU runtime, communicator).  Kept separate so that
each native translation unit has its Python declaration next to the others."""
import ctypes as C

vp, sz, i, f = C.c_void_p, C.c_size_t, C.c_int, C.c_float
ll = C.c_longlong
cs = C.c_char_p

PROTOTYPES = {
    # csrc/gpu/train_kernels.cu
    "cclx_sq_norm": (i, [vp, sz, i, vp, vp, vp]),
    "cclx_adamw_flat": (i, [vp, vp, i, vp, vp, vp, sz, sz, f, f, f, f, f, i, f, f, vp, vp]),
    "cclx_softmax_xent": (i, [vp, vp, vp, sz, i, sz, f, i, vp]),
    # csrc/gpu/moe_kernels.cu
    "cclx_moe_gather_rows": (i, [vp, vp, vp, sz, i, vp]),
    "cclx_moe_combine": (i, [vp, vp, vp, vp, sz, i, i, vp]),
    "cclx_moe_dispatch": (i, [vp, vp, vp, vp, vp, sz, i, i, vp, sz, vp, i, vp]),
    "cclx_moe_combine_peer": (i, [vp, vp, vp, vp, vp, vp, sz, i, i, vp, i, vp]),
    # csrc/capi/capi_comm.cpp
    "cclx_kvs_create_main": (vp, [cs]),
    "cclx_kvs_create_peer": (vp, [cs]),
    "cclx_kvs_address": (i, [vp, vp, sz]),
    "cclx_kvs_set": (i, [vp, cs, vp, sz]),
    "cclx_kvs_get": (ll, [vp, cs, vp, sz, i]),
    "cclx_kvs_add": (ll, [vp, cs, ll]),
    "cclx_kvs_count": (ll, [vp, cs]),
    "cclx_kvs_del": (i, [vp, cs]),
    "cclx_kvs_barrier": (i, [vp, cs, i, i]),
    "cclx_kvs_destroy": (i, [vp]),
    "cclx_comm_create": (vp, [i, i, vp]),
    "cclx_comm_split": (vp, [vp, i, i]),
    "cclx_comm_node": (vp, [vp]),
    "cclx_comm_r2r": (vp, [vp]),
    "cclx_comm_rank": (i, [vp]),
    "cclx_comm_size": (i, [vp]),
    "cclx_comm_id": (ll, [vp]),
    "cclx_comm_local_rank": (i, [vp]),
    "cclx_comm_local_size": (i, [vp]),
    "cclx_comm_device": (vp, [vp]),
    "cclx_comm_release_device": (i, [vp]),
    "cclx_comm_abort": (i, [vp]),
    "cclx_comm_heartbeat": (i, [vp]),
    "cclx_comm_peer_alive": (i, [vp, i, i]),
    "cclx_comm_destroy": (i, [vp]),
    "cclx_comm_cache_size": (ll, [vp]),
    "cclx_coll": (vp, [vp, vp]),
    "cclx_event_wait": (i, [vp]),
    "cclx_event_test": (i, [vp]),
    "cclx_event_native": (vp, [vp]),
    "cclx_event_destroy": (i, [vp]),
    "cclx_group_start": (i, []),
    "cclx_group_end": (i, []),
    "cclx_fusion_flush": (i, []),
    "cclx_datatype_create": (i, [sz]),
    "cclx_datatype_free": (i, [i]),
    "cclx_datatype_size": (ll, [i]),
    "cclx_comp_reduce": (i, [vp, sz, vp, i, i]),
    "cclx_comp_impl": (cs, [i]),
    "cclx_select_cpu_algo": (i, [i, sz, i, vp, sz]),
    "cclx_selector_reload": (i, []),
    "cclx_parse_algo_spec": (i, [i, cs]),
    "cclx_stats": (ll, [i, i]),
    "cclx_topo_describe": (i, [vp, sz]),
    "cclx_numa_query": (i, [C.c_char_p, i, i, C.c_char_p, C.POINTER(C.c_int), i]),
    "cclx_numa_auto_worker_cpus": (i, [C.POINTER(C.c_int), i, i, i, i, C.POINTER(C.c_int)]),
    "cclx_numa_selftest": (i, [i, sz]),
    "cclx_env_size": (i, [cs, C.POINTER(sz)]),
}
