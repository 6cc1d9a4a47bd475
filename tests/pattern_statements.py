"""One or more statements for every instruction pattern of the reference grammar (ptx_parser/src/lib.rs:2093-4462),
written from the pattern heads and rule lines there.  Shared by the oracle pin test and the GPU test."""

STATEMENTS = [
    # mov, st (2093-2186)
    "mov.u32 %r1, %r2;", "mov.v2.f32 %f1, {%f2, %f3};", "mov.pred %p1, %p2;",
    "st.global.u32 [%rd1], %r1;", "st.weak.shared.cg.v4.f32 [%rd1+16], {%f1,%f2,%f3,%f4};", "st.global.L1::evict_last.L2::cache_hint.u64 [%rd1], %rd2, %rd3;",
    "st.volatile.global.v2.u32 [%rd1], {%r1,%r2};", "st.relaxed.gpu.global.u32 [%rd1], %r1;", "st.release.sys.shared.b64 [%rd1], %rd2;",
    "st.mmio.relaxed.sys.global.u32 [%rd1], %r1;",
    # ld (2187-2310)
    "ld.global.u32 %r1, [%rd1];", "ld.weak.shared.v2.f32 {%f1,%f2}, [%rd1+8];", "ld.const.ca.L1::evict_first.L2::128B.u8 %r1, [%rd1];",
    "ld.param.u64 %rd1, [p0].unified;", "ld.volatile.shared.L2::64B.u32 %r1, [%rd1];", "ld.relaxed.cta.global.f32 %f1, [%rd1];",
    "ld.acquire.sys.global.L2::256B.v4.u32 {%r1,%r2,%r3,%r4}, [%rd1];", "ld.mmio.relaxed.sys.global.u32 %r1, [%rd1];",
    "ld.global.nc.u32 %r1, [%rd1];", "ld.global.ca.nc.L1::no_allocate.L2::cache_hint.v2.f32 {%f1,%f2}, [%rd1], %rd9;",
    # add (2311-2448)
    "add.u32 %r1, %r2, %r3;", "add.s64 %rd1, %rd2, %rd3;", "add.sat.s32 %r1, %r2, %r3;", "add.s32 %r1, %r2, 5;", "add.rn.ftz.sat.f32 %f1, %f2, %f3;",
    "add.f32 %f1, %f2, 0f3F800000;", "add.rz.f64 %fd1, %fd2, %fd3;", "add.rn.ftz.f16 %h1, %h2, %h3;", "add.f16x2 %r1, %r2, %r3;", "add.rn.bf16 %h1, %h2, %h3;",
    "add.bf16x2 %r1, %r2, %r3;",
    # mul (2449-2566)
    "mul.lo.s32 %r1, %r2, %r3;", "mul.hi.u64 %rd1, %rd2, %rd3;", "mul.wide.u32 %rd1, %r2, %r3;", "mul.wide.s16 %r1, %h2, %h3;", "mul.rn.ftz.f32 %f1, %f2, %f3;",
    "mul.rm.f64 %fd1, %fd2, %fd3;", "mul.f16 %h1, %h2, %h3;", "mul.rn.sat.f16x2 %r1, %r2, %r3;", "mul.bf16 %h1, %h2, %h3;", "mul.rn.bf16x2 %r1, %r2, %r3;",
    # set, setp (2567-2648)
    "set.lt.u32.s32 %r1, %r2, %r3;", "set.ge.ftz.f32.f32 %f1, %f2, %f3;", "set.eq.f16x2.f16x2 %r1, %r2, %r3;", "set.ne.and.u32.u32 %r1, %r2, %r3, !%p1;",
    "setp.lt.s32 %p1, %r1, %r2;", "setp.hi.u32 %p1|%p2, %r1, %r2;", "setp.gtu.ftz.f32 %p1, %f1, %f2;", "setp.eq.and.b32 %p1|%p2, %r1, %r2, %p3;",
    "setp.ge.or.f64 %p1, %fd1, %fd2, !%p3;",
    # not or and bra call cvt (2649-2751)
    "not.b32 %r1, %r2;", "not.pred %p1, %p2;", "or.b64 %rd1, %rd2, %rd3;", "or.pred %p1, %p2, %p3;", "and.b16 %h1, %h2, %h3;", "and.b32 %r1, %r2, 255;",
    "bra L1;", "bra.uni L2;", "@%p1 bra L1;", "@!%p2 bra.uni L1;",
    "cvt.rn.f32.s32 %f1, %r1;", "cvt.rzi.ftz.s32.f32 %r1, %f1;", "cvt.f64.f32 %fd1, %f1;", "cvt.u16.u32 %h1, %r2;", "cvt.sat.u8.s32 %r1, %r2;", "cvt.s64.s32 %rd1, %r1;",
    "cvt.rn.f16.f32 %h1, %f1;", "cvt.rz.relu.bf16x2.f32 %r1, %f1, %f2;", "cvt.rn.satfinite.f16x2.f32 %r1, %f1, %f2;", "cvt.rn.f16x2.e4m3x2 %r1, %h1;",
    "cvt.rn.satfinite.e4m3x2.f32 %h1, %f1, %f2;", "cvt.rn.satfinite.relu.e5m2x2.f32 %h1, %f1, %f2;", "cvt.pack.sat.u8.s32.b32 %r1, %r2, %r3, %r4;",
    # shl shr cvta abs (2752-2893)
    "shl.b32 %r1, %r2, 3;", "shr.s32 %r1, %r2, %r3;", "shr.u64 %rd1, %rd2, 7;", "cvta.global.u64 %rd1, %rd2;", "cvta.shared.u32 %r1, %r2;", "cvta.to.local.u64 %rd1, %rd2;",
    "abs.s32 %r1, %r2;", "abs.ftz.f32 %f1, %f2;", "abs.f64 %fd1, %fd2;", "abs.f16 %h1, %h2;", "abs.ftz.f16x2 %r1, %r2;", "abs.bf16 %h1, %h2;", "abs.bf16x2 %r1, %r2;",
    # mad fma sub (2894-3168)
    "mad.lo.s32 %r1, %r2, %r3, %r4;", "mad.hi.u64 %rd1, %rd2, %rd3, %rd4;", "mad.wide.u16 %r1, %h2, %h3, %r4;", "mad.hi.sat.s32 %r1, %r2, %r3, %r4;",
    "mad.ftz.f32 %f1, %f2, %f3, %f4;", "mad.rn.sat.f32 %f1, %f2, %f3, %f4;", "mad.rz.f64 %fd1, %fd2, %fd3, %fd4;",
    "fma.rn.ftz.f32 %f1, %f2, %f3, %f4;", "fma.rp.f64 %fd1, %fd2, %fd3, %fd4;", "fma.rn.sat.f16 %h1, %h2, %h3, %h4;", "fma.rn.relu.bf16x2 %r1, %r2, %r3, %r4;",
    "fma.rn.f16x2 %r1, %r2, %r3, %r4;",
    "sub.u16 %h1, %h2, %h3;", "sub.sat.s32 %r1, %r2, %r3;", "sub.rn.ftz.f32 %f1, %f2, %f3;", "sub.rz.f64 %fd1, %fd2, %fd3;", "sub.sat.f16 %h1, %h2, %h3;",
    "sub.rn.f16x2 %r1, %r2, %r3;", "sub.bf16 %h1, %h2, %h3;", "sub.rn.bf16x2 %r1, %r2, %r3;",
    # min max (3169-3377)
    "min.u32 %r1, %r2, %r3;", "min.s16x2 %r1, %r2, %r3;", "min.s64 %rd1, %rd2, %rd3;", "min.ftz.NaN.f32 %f1, %f2, %f3;", "min.f64 %fd1, %fd2, %fd3;", "min.NaN.f16 %h1, %h2, %h3;",
    "min.ftz.f16x2 %r1, %r2, %r3;", "min.bf16 %h1, %h2, %h3;", "min.NaN.bf16x2 %r1, %r2, %r3;",
    "max.s32 %r1, %r2, %r3;", "max.u16x2 %r1, %r2, %r3;", "max.u64 %rd1, %rd2, %rd3;", "max.NaN.f32 %f1, %f2, %f3;", "max.f64 %fd1, %fd2, %fd3;", "max.ftz.f16 %h1, %h2, %h3;",
    "max.f16x2 %r1, %r2, %r3;", "max.NaN.bf16 %h1, %h2, %h3;", "max.bf16x2 %r1, %r2, %r3;",
    # rcp sqrt rsqrt selp (3378-3489)
    "rcp.approx.ftz.f32 %f1, %f2;", "rcp.approx.ftz.f64 %fd1, %fd2;", "rcp.rn.f32 %f1, %f2;", "rcp.rz.f64 %fd1, %fd2;", "sqrt.approx.f32 %f1, %f2;", "sqrt.rn.ftz.f32 %f1, %f2;",
    "sqrt.rm.f64 %fd1, %fd2;", "rsqrt.approx.ftz.f32 %f1, %f2;", "rsqrt.approx.f64 %fd1, %fd2;", "rsqrt.approx.ftz.f64 %fd1, %fd2;", "selp.f32 %f1, %f2, %f3, %p1;",
    "selp.b64 %rd1, %rd2, %rd3, %p1;",
    # barrier bar atom (3490-3646)
    "barrier.sync 0;", "barrier.cta.sync.aligned %r1, %r2;", "bar.sync 1;", "bar.cta.sync 2, 128;", "bar.red.popc.u32 %r1, 0, %p1;", "bar.cta.red.and.pred %p1, 1, 64, !%p2;",
    "bar.red.or.pred %p1, 0, %p2;", "bar.warp.sync 0xffffffff;",
    "atom.global.add.u32 %r1, [%rd1], %r2;", "atom.acq_rel.sys.shared.max.s32 %r1, [%rd1], %r2;", "atom.min.u64 %rd1, [%rd2], %rd3;", "atom.global.inc.u32 %r1, [%rd1], %r2;",
    "atom.relaxed.cta.global.exch.b32 %r1, [%rd1], %r2;", "atom.global.add.L2::cache_hint.f32 %f1, [%rd1], %f2, %rd9;", "atom.global.and.b64 %rd1, [%rd2], %rd3;",
    "atom.acquire.gpu.global.cas.b32 %r1, [%rd1], %r2, %r3;", "atom.shared.cas.b64 %rd1, [%rd2], %rd3, %rd4;", "atom.global.exch.b128 %q1, [%rd1], %q2;",
    "atom.global.add.v2.f32 {%f1,%f2}, [%rd1], {%f3,%f4};", "atom.global.add.noftz.f16 %h1, [%rd1], %h2;", "atom.global.max.noftz.v2.bf16 {%h1,%h2}, [%rd1], {%h3,%h4};",
    "atom.global.add.noftz.f16x2 %r1, [%rd1], %r2;", "atom.global.min.noftz.v4.bf16x2 {%r1,%r2,%r3,%r4}, [%rd1], {%r5,%r6,%r7,%r8};",
    # div neg sin cos lg2 ex2 (3647-3854)
    "div.s32 %r1, %r2, %r3;", "div.u64 %rd1, %rd2, %rd3;", "div.approx.ftz.f32 %f1, %f2, %f3;", "div.full.f32 %f1, %f2, %f3;", "div.rn.f32 %f1, %f2, %f3;", "div.rz.f64 %fd1, %fd2, %fd3;",
    "neg.s32 %r1, %r2;", "neg.ftz.f32 %f1, %f2;", "neg.f64 %fd1, %fd2;", "neg.f16 %h1, %h2;", "neg.ftz.f16x2 %r1, %r2;", "neg.bf16 %h1, %h2;", "neg.bf16x2 %r1, %r2;",
    "sin.approx.ftz.f32 %f1, %f2;", "cos.approx.f32 %f1, %f2;", "lg2.approx.f32 %f1, %f2;", "ex2.approx.ftz.f32 %f1, %f2;", "ex2.approx.f16 %h1, %h2;", "ex2.approx.f16x2 %r1, %r2;",
    "ex2.approx.ftz.bf16 %h1, %h2;", "ex2.approx.ftz.bf16x2 %r1, %r2;",
    # clz .. bfind (3855-4462)
    "clz.b32 %r1, %r2;", "clz.b64 %r1, %rd2;", "brev.b32 %r1, %r2;", "popc.b64 %r1, %rd2;", "xor.b32 %r1, %r2, %r3;", "xor.pred %p1, %p2, %p3;", "rem.s32 %r1, %r2, %r3;", "rem.u64 %rd1, %rd2, %rd3;",
    "bfe.u32 %r1, %r2, %r3, %r4;", "bfe.s64 %rd1, %rd2, %r3, %r4;", "bfi.b32 %r1, %r2, %r3, %r4, %r5;", "bmsk.clamp.b32 %r1, %r2, %r3;", "bmsk.wrap.b32 %r1, %r2, %r3;",
    "prmt.b32 %r1, %r2, %r3, %r4;", "activemask.b32 %r1;", "membar.cta;", "membar.sys;", "membar.gl;", "ret;", "ret.uni;",
    "mul24.lo.s32 %r1, %r2, %r3;", "mul24.hi.u32 %r1, %r2, %r3;", "shfl.bfly.b32 %r1, %r2, 1, 31;", "shfl.up.b32 %r1|%p1, %r2, %r3, %r4;",
    "shfl.sync.bfly.b32 %r1|%p1, %r2, 1, 31, -1;", "shfl.sync.idx.b32 %r1, %r2, %r3, 31, 0xffffffff;", "nanosleep.u32 %r1;", "nanosleep.u32 100;",
    "tanh.approx.f32 %f1, %f2;", "tanh.approx.f16x2 %r1, %r2;",
    "cp.async.ca.shared.global [%rd1], [%rd2], 4;", "cp.async.cg.shared.global.L2::128B [%rd1], [%rd2], 16, %r1;", "cp.async.ca.shared.global.L2::cache_hint [%rd1], [%rd2], 8, 4, %rd9;",
    "cp.async.ca.shared.global [%rd1], [%rd2], 3;",
    "cp.async.commit_group;", "cp.async.wait_group 2;", "cp.async.wait_all;", "shf.l.clamp.b32 %r1, %r2, %r3, %r4;", "shf.r.wrap.b32 %r1, %r2, %r3, 5;", "trap;", "exit;",
    "dp4a.u32.s32 %r1, %r2, %r3, %r4;", "dp4a.s32.s32 %r1, %r2, %r3, %r4;", "vote.sync.all.pred %p1, %p2, 0xffffffff;", "vote.sync.any.pred %p1, !%p2, %r1;",
    "vote.ballot.b32 %r1, %p1;", "vote.sync.ballot.b32 %r1, !%p1, 0xffffffff;", "redux.sync.add.s32 %r1, %r2, 0xffffffff;", "redux.sync.or.b32 %r1, %r2, %r3;", "redux.sync.max.u32 %r1, %r2, -1;",
    "ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%r1,%r2,%r3,%r4}, [%rd1];", "ldmatrix.sync.aligned.m8n8.x1.b16 {%r1}, [%rd1];", "ldmatrix.sync.aligned.m8n8.x2.shared::cta.b16 {%r1,%r2}, [%rd1];",
    "griddepcontrol.launch_dependents;", "griddepcontrol.wait;",
    "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%f1,%f2,%f3,%f4}, {%r1,%r2,%r3,%r4}, {%r5,%r6}, {%f5,%f6,%f7,%f8};",
    "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%f1,%f2,%f3,%f4}, {%r1,%r2,%r3,%r4}, {%r5,%r6}, {%f5,%f6,%f7,%f8};",
    "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%r1,%r2,%r3,%r4}, {%r5,%r6,%r7,%r8}, {%r9,%r10}, {%r11,%r12,%r13,%r14};",
    "copysign.f32 %f1, %f2, %f3;", "copysign.f64 %fd1, %fd2, %fd3;", "prefetch.global.L1 [%rd1];", "prefetch.L2 [%rd1];", "prefetch.local.L2 [%rd1];",
    "createpolicy.fractional.L2::evict_last.b64 %rd1;", "createpolicy.fractional.L2::evict_first.b64 %rd1, 0.5;", "createpolicy.fractional.L2::evict_normal.b64 %rd1, 1.0;",
    "sad.u32 %r1, %r2, %r3, %r4;", "sad.s64 %rd1, %rd2, %rd3, %rd4;", "dp2a.lo.u32.s32 %r1, %r2, %r3, %r4;", "dp2a.hi.s32.u32 %r1, %r2, %r3, %r4;",
    "add.cc.u32 %r1, %r2, %r3;", "addc.s32 %r1, %r2, %r3;", "addc.cc.u64 %rd1, %rd2, %rd3;", "sub.cc.s32 %r1, %r2, %r3;", "subc.u32 %r1, %r2, %r3;", "subc.cc.s64 %rd1, %rd2, %rd3;",
    "mad.lo.cc.u32 %r1, %r2, %r3, %r4;", "mad.hi.cc.s32 %r1, %r2, %r3, %r4;", "madc.lo.u32 %r1, %r2, %r3, %r4;", "madc.hi.cc.u64 %rd1, %rd2, %rd3, %rd4;",
    "vshr.u32.u32.u32.clamp.add %r1, %r2, %r3, %r4;", "vshr.u32.u32.u32.wrap.add %r1, %r2, %r3, %r4;",
    "tex.1d.v4.f32.s32 {%f1,%f2,%f3,%f4}, [tex0, {%r1}];", "tex.2d.v4.u32.f32 {%r1,%r2,%r3,%r4}, [tex0, {%f1,%f2}];", "tex.3d.v4.s32.s32 {%r1,%r2,%r3,%r4}, [tex0, {%r5,%r6,%r7,%r8}];",
    "match.any.sync.b32 %r1, %r2, 0xffffffff;", "match.any.sync.b64 %r1, %rd2, %r3;", "bfind.u32 %r1, %r2;", "bfind.shiftamt.u32 %r1, %r2;", "bfind.s64 %r1, %rd2;",
    "call foo, (%r1);", "call.uni (%r1), bar, (%r2, %r3);",
]

DECLS = (".reg .b32 %r<20>; .reg .b64 %rd<10>; .reg .f32 %f<10>; .reg .f64 %fd<6>; .reg .b16 %h<6>; .reg .pred %p<6>; .reg .b128 %q<3>;")
HEADER = ".version 8.5\n.target sm_90\n.address_size 64\n"
PRELUDE = ".func foo(.param .b32 a)\n;\n.func (.param .b32 r) bar(.param .b32 a, .param .b32 b)\n;\n.global .texref tex0;\n"


def module(statements):
    return HEADER + PRELUDE + ".visible .entry k(.param .u64 p0)\n{\n" + DECLS + "\nL1:\nL2:\n" + "\n".join(statements) + "\nret;\n}\n"
