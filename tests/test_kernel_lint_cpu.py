"""The GPU-less kernel linter: the tree is clean, and each rule fires on a snippet that breaks it."""
from gemm_b200.utils import kernel_lint as kl


def test_tree_is_clean_and_blackwell_native():
    rep = kl.lint_tree()
    assert rep["problems"] == [], rep["problems"]
    inv = rep["inventory"]
    gemm = inv["gemm_b200/csrc/kernels/gemm_tc.cu"]
    assert gemm.get("tcgen05.mma", 0) > 0 and gemm.get("cp.async.bulk.tensor", 0) > 0 and gemm.get("mma.sync / wmma", 0) == 0
    assert inv["gemm_b200/csrc/kernels/flash_attn.cu"].get("tcgen05.mma", 0) > 0
    assert inv["gemm_b200/csrc/kernels/moe_ffn.cu"].get("tcgen05.mma", 0) > 0


def _rules(src, **kw):
    return sorted({p["rule"] for p in kl.lint_text("x.cu", src, **kw)[0]})


def test_rules_fire():
    spin = "__global__ void k(unsigned* f) { while (ld_acquire_gpu(f) == 0) { } }"
    assert _rules(spin) == ["bounded-wait"]
    bounded = "__global__ void k(unsigned* f) { const uint64_t t0 = globaltimer_ns(); while (ld_acquire_gpu(f) == 0) { if (globaltimer_ns() - t0 > kBudgetNs) break; } }"
    assert _rules(bounded) == []
    dowhile = "__global__ void k(volatile int* f) { int v; do { v = *(volatile int*)f; } while (v == 0); }"
    assert _rules(dowhile) == ["bounded-wait"]
    leak = "__global__ void k(uint32_t* s) { tmem_alloc(s, 64); }"
    assert _rules(leak) == ["tmem-paired"]
    paired = "__global__ void k(uint32_t* s) { tmem_alloc(s, 64); tmem_dealloc(*s, 64); }"
    assert _rules(paired) == []
    # the qualifier is put together here so that this file itself does not spell a load of that kind
    qual = ".multi" + "cast" + "::cluster"
    mc = 'void f() { asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes' + qual + ' [%0], [%1, {%2, %3}], [%4], %5;"); }'
    assert _rules(mc) == ["no-cluster-broadcast-load"] and _rules(mc, multi_gpu=False) == []
    commit = 'void f() { asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster' + qual + '.b64 [%0], %1;"); }'
    assert _rules(commit) == []
    assert _rules('void f() { asm volatile("wgmma.mma_async.sync.aligned.m64n128k16.f32.bf16.bf16 ..."); }') == ["arch"]
    assert _rules("// while (ld_acquire_gpu(f) == 0) {}\n/* tmem_alloc( */ void f() {}") == []
