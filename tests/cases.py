"""Edge-case inputs shared by the CPU (emulated pipeline) and GPU parity tests.  Each is a complete module text."""
HEADER = ".version 6.5\n.target sm_30\n.address_size 64\n"
DECLS = ".reg .b32 %r<10>; .reg .b64 %rd<10>; .reg .f32 %f<10>; .reg .f64 %fd<4>; .reg .pred %p<4>;"


def body(stmts):
    return HEADER + ".visible .entry k()\n{\n" + DECLS + "\n" + stmts + "\nret;\n}\n"


LITERALS = ["10", "18446744073709551615", "18446744073709551616", "10U", "-10U", "-9223372036854775808",
            "-9223372036854775809", "010", "09", "0", "0x1F", "0X1f", "0xFFFFFFFFFFFFFFFF", "0xFFU", "0xU", "0xZZ",
            "0f3F800000", "0fGGGGGGGG", "0d3FF0000000000000", "1.5", ".5", "1.5e-3", "0.1", "1.7976931348623157e308",
            "4.9e-324", "1.0e400", "WARP_SZ", "2.4703282292062327e-324", "2.4703282292062328e-324",
            "9007199254740993.0", "9007199254740992.9999999999999999999999", "8.98846567431158e307"]

STATEMENTS = [
    "mov.f64 %fd1, -1.5;", "mov.f32 %f1, -0f3F800000;", "mov.f32 %f1, 0f3F8000;", "mov.f64 %fd1, 2.E5;", "mov.f64 %fd1, 2.;",
    "bra add;", ".reg .b32 %z<0>;", ".reg .b32 %a, %b<4>;", "ld.u32.v2 {%r1,%r2}, [%rd1];", "add.s32.s32 %r1, %r2, %r3;",
    "shf.l.wrap.b32 %r1, %r2.r, %r3, %r4;", "cvt.f32.u32 %f1, %r1;", "setp.lt.ftz.u32 %p1, %r1, %r2;",
    "setp.ltu.u32 %p1, %r1, %r2;", "add:\n", ".reg .b32 %q<99999999999>;", "mov.u32 %r1, %v.q;",
    "ld.global.u32 %r1, [%rd1+2147483648];", "mov.u32 foo, {} {};", "ret }", "{ add.s32 %r1,%r2,%r3; { ret } }",
    "{ { foo bar } ret; } ret;", "mov.b32 %r1, %envreg3;", ".loc 1 2 3\n}", "@%p1 bra L1; L1:",
    "@!%p1 add.s32 %r1,%r2,%r3;", "foo: bar: ret;", ".pragma \"nounroll\";",
    "unknown_op1.asdf foobar;\nadd.u64 %rd1,%rd2,1;\nunknown_op2 t, u;",
    "ld.global.nc.ca.L1::evict_last.u32 %r1, [%rd1];", "ld.global.L2::cache_hint.u32 %r1, [%rd1], %rd2;",
    "cp.async.ca.shared.global [%rd1], [%rd2], 16;", "cp.async.ca.shared.global [%rd1], [%rd2], 5, 4;",
    "createpolicy.fractional.L2::evict_last.b64 %rd1, 0.5;", "createpolicy.fractional.L2::evict_last.b64 %rd1;",
    "bar.red.and.pred %p1, 0, !%p2;", "bar.red.or.pred %p1, 0, 32, %p2;", "barrier.sync.aligned 0, 32;",
    "shfl.sync.bfly.b32 %r1|%p1, %r2, 1, 31, -1;", "shfl.bfly.b32 %r1, %r2, 1, 31;",
    "vote.sync.ballot.b32 %r1, !%p1, -1;", "vote.ballot.b32 %r1, %p1;", "vshr.u32.u32.u32.clamp.add %r1, %r2, %r3, %r4;",
    "tex.2d.v4.f32.f32 {%f1,%f2,%f3,%f4}, [tex, {%f5,%f6}];", "atom.global.add.u32 %r1, [%rd1], 1;",
    "atom.acq_rel.gpu.global.cas.b32 %r1, [%rd1], %r2, %r3;", "atom.global.add.noftz.f16x2 %r1, [%rd1], %r2;",
    "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%f1,%f2,%f3,%f4}, {%r1,%r2,%r3,%r4}, {%r5,%r6}, {%f5,%f6,%f7,%f8};",
    "cvt.rn.satfinite.e4m3x2.f32 %r1, %f1, %f2;", "cvt.rn.f16x2.f32 %r1, %f1, %f2;", "cvt.sat.u8.s32 %r1, %r2;",
    "cvt.f64.f32 %fd1, %f1;", "cvt.rn.f64.f32 %fd1, %f1;", "cvt.pred.u32 %p1, %r1;", "membar.gl;", "membar.sys;",
    "ld.volatile.shared.v2.f32 {%f1,%f2}, [%rd1];", "st.release.sys.global.u32 [%rd1], %r1;", "st.mmio.relaxed.sys.u32 [%rd1], %r1;",
    "lg2.f32.ftz.approx %f1, %f2;", "rsqrt.approx.ftz.f64 %fd1, %fd2;", "min.NaN.f32 %f1, %f2, %f3;",
    "mad.hi.sat.s32 %r1, %r2, %r3, %r4;", "mad.lo.cc.u32 %r1, %r2, %r3, %r4;", "madc.hi.cc.u32 %r1, %r2, %r3, %r4;",
    "prefetch.global.L2 [%rd1];", "ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%r1,%r2,%r3,%r4}, [%rd1];",
    "griddepcontrol.wait;", "redux.sync.add.s32 %r1, %r2, -1;", "match.any.sync.b32 %r1, %r2, -1;", "trap;", "exit;",
    "ret.uni;", "bra.uni L;", "nanosleep.u32 100;", "activemask.b32 %r1;", "bfind.shiftamt.u32 %r1, %r2;",
    "dp2a.lo.u32.s32 %r1, %r2, %r3, %r4;", "set.lt.and.ftz.u32.f32 %r1, %f1, %f2, !%p1;", "setp.eq.and.b32 %p1|%p2, %r1, %r2, %p3;",
    "mov.b32 %r1, %r2+4;", "mov.b32 %r1, [%r2];", "st.global.u32 [%rd1+-4], %r1;", "ld.param.u64 %rd1, [k_param_0];",
    ".local .align 8 .b8 buf[16];", ".shared .v2 .f32 sm;", ".param .b32 pp;", ".global .u32 gg = 5;", ".reg .v4 .f32 %vec, %vec2;",
]

MODULES = [
    ".version 6.5\n.target sm_90ab\n", ".version 6.5 .target sm_30, debug", HEADER + "#", HEADER + "/* never",
    HEADER + "\"open", HEADER + ".visible .entry k() { # ret; }", "", "// only comment\n",
    ".version 6.5\n.target sm_30\n.address_size 16\n.visible .entry k() { ret; }",
    ".version 0d401F333333333333\n.target sm_30\n", ".version 6.5\n.target add\n", ".version 65\n.target sm_30\n",
    HEADER + ".global .bad_type foo;\n.const .b32 bar;\n",
    HEADER + ".broken_directive_fail; 34; {\n.visible .entry add(.param .u64 input)\n{\n ret;\n}\nsection foobar }",
    HEADER + ".global .b32 global[4] = {  unknown (1),   2,   3,   4};\n.visible .entry func1()\n{\nst.u64 [out_addr], temp2;\nret;\n}\n"
             ".visible .entry func1()\n{\nbroken_instruction;\nret;\n}",
    HEADER + ".func (.reg .b32 r) f(.reg .b32 a, .reg .b32 b);\n.visible .entry k()\n{\n .reg .b32 %r<4>;\n call (%r1), f, (%r2, %r3);\n"
             " call (%r1), f, (%r2);\n call g;\n call.uni k;\n ret;\n}\n",
    HEADER + ".func (.reg .b32 r) f(.reg .b32 a, .reg .b32 b)\n{\n ret;\n}\n.func f(.reg .b32 a);\n.visible .entry k()\n{\n"
             " .reg .b32 %r<4>;\n call (%r1), f, (%r2, %r3);\n call f, (%r2);\n ret;\n}\n",
    HEADER + ".func f(.reg .b32 a)\n{\n call f, (a);\n ret;\n}\n.func f(.reg .b32 a)\n{\n call f, (a);\n ret;\n}\n",
    HEADER + ".const .align 4 .b8 constData[8];\n.global .s32 x[4] = {1};\n.global .f32 y[2] = {0f3F800000};\n.global .b32 z<4>;\n"
             ".extern .shared .b8 sh[];\n.global .texref tex;\n.global .v2 .f32 vv = 1.0;\n.global .b8 e[2] = {};\n.global .u32 a[2][2];",
    HEADER + ".file 1 \"a.cu\"\n.file 2 \"b.cu\", 123, 456\n.section .debug_abbrev\n{\n.b8 1\n.b8 17, 2\n.b32 .debug_info\nlbl:\n.b64 foo\n}\n"
             ".visible .entry k() { ret; }",
    HEADER + ".visible .entry k(.param .u64 .ptr .global .align 8 p, .param .align 4 .b8 q[16])\n.maxntid 128, 1\n.minnctapersm 2\n{\n ret;\n}",
    HEADER + ".visible .entry k() { ret; } garbage", HEADER + ".visible .entry k() { ret; } garbage more",
    HEADER + ".visible .entry k() { ret;", HEADER + "}", HEADER + ".visible .entry k() { ret; } }",
    HEADER + ".weak .func w() { ret; }\n.extern .func e();\n.visible .func (.param .align 16 .b8 r[32]) g(.param .b64 a) .noreturn;",
    HEADER + ".visible .entry k()\n{\n .reg .b32 %r<4>;\n {\n  .reg .b32 %t;\n  {\n   add.s32 %t, %r1, %r2;\n  }\n }\n ret;\n}",
    HEADER + ".visible .entry k() { ld.global.u32 %r1, [%rd1]; .global .u32 inner; bogus }\n.global .u32 after;",
    HEADER + ".visible .entry " + "k" * 300 + "() { ret; }",
    HEADER + "// c1\n/* c2 */ .visible /* mid */ .entry k() // tail\n{ ret; /* x */ }\n/**/",
    HEADER + ".visible .entry k() { mov.u32 %r1, 0x" + "F" * 200 + "; ret; }",
]


def all_cases():
    out = [body("mov.b64 %rd1, " + lit + ";") for lit in LITERALS]
    out += [body(s) for s in STATEMENTS]
    out += MODULES
    return out


def class_cases():
    """Statements of one shape that must NOT share a record template: the decoder's path depends on a token's text
    (dot-identifiers, %envreg names), on what kind of number a literal is (suffix, radix errors, which limits its
    magnitude exceeds) or on its surroundings; and statements of one shape that must share one: only names and the
    digits of literals differ, and the template is instantiated with each statement's own values.
    Every module repeats each statement, so that all but the first meet an existing class."""
    groups = [
        # same kinds, different identifier spellings and lengths: one class, records differ in offsets and lengths only
        ["add.s32 %r1, %r2, %r3;", "add.s32 %rd10, %a, %bb;", "add.s32 %r1,%r2,%r3;", "add.s32   %x ,\n %yy , %zzz ;"],
        # the digits of a number are not part of the class, the facts the grammar can learn from them are: one template
        # serves 1, 2, 0x2, 02 and 077; the suffix, the limits and conversion errors make classes of their own
        ["mov.u32 %r1, 1;", "mov.u32 %r1, 2;", "mov.u32 %r1, 0x2;", "mov.u32 %r1, 02;", "mov.u32 %r1, 077;", "mov.u32 %r1, 2U;",
         "mov.u32 %r1, 99999999999;", "mov.u32 %r1, 2147483647;", "mov.u32 %r1, 2147483648;", "mov.u32 %r1, 4294967295;",
         "mov.u32 %r1, 4294967296;", "mov.u64 %rd1, 9223372036854775807;", "mov.u64 %rd1, 9223372036854775808;",
         "mov.u64 %rd1, 18446744073709551615;", "mov.u64 %rd1, 18446744073709551616;", "mov.u64 %rd1, 18446744073709551615U;",
         "mov.u64 %rd1, 0xFFFFFFFFFFFFFFFF;", "mov.u64 %rd1, 0x1FFFFFFFFFFFFFFFF;", "mov.u32 %r1, 09;", "mov.u32 %r1, 0xG;", "mov.u32 %r1, 0xU;",
         "mov.s64 %rd1, -1;", "mov.s64 %rd1, -9223372036854775807;", "mov.s64 %rd1, -9223372036854775808;", "mov.s64 %rd1, -9223372036854775809;",
         "mov.s64 %rd1, -0x10;", "mov.s64 %rd1, -5U;", "mov.s64 %rd1, -18446744073709551616;", "mov.u32 %r1, WARP_SZ;"],
        ["mov.f32 %f1, 0f3F800000;", "mov.f32 %f1, 0f40000000;", "mov.f32 %f1, 0fBF80000a;", "mov.f32 %f1, 0f3F80000G;", "mov.f64 %fd1, 1.5;",
         "mov.f64 %fd1, 1.5e3;", "mov.f64 %fd1, 2.5e-3;", "mov.f64 %fd1, .5;", "mov.f64 %fd1, 8.98846567431158e307;", "mov.f64 %fd1, 1.0e400;",
         "mov.f64 %fd1, 0d3FF0000000000000;", "mov.f64 %fd1, 0dBFF000000000000Z;", "mov.f64 %fd1, 0d4000000000000000;", "mov.f64 %fd1, -1.5;"],
        ["ld.global.u32 %r1, [%rd1+4];", "ld.global.u32 %r1, [%rd1+8];", "ld.global.u32 %r1, [%rd1+-4];", "ld.global.u32 %r1, [%rd1+-8];",
         "ld.global.u32 %r1, [%rd1];", "ld.global.u32 %r1, [%rd1+0x7FFFFFFF];", "ld.global.u32 %r1, [%rd1+2147483648];",
         "ld.global.u32 %r1, [%rd1+-2147483647];", "ld.global.u32 %r1, [%rd1+-2147483648];", "ld.global.u32 %r1, [%rd1+010];",
         "ld.global.u32 %r1, [%rd1+16U];", "st.shared.v2.f32 [%rd2+64], {%f1, 0f3F800000};", "st.shared.v2.f32 [%rd2+128], {%f1, 0f40000000};",
         "shfl.sync.bfly.b32 %r1|%p1, %r2, 1, 31, -1;", "shfl.sync.bfly.b32 %r1|%p1, %r2, 16, 0x1f, -2;", "bar.sync 0;", "bar.sync 15;"],
        # vector members and unknown dot words
        ["mov.u32 %r1, %tid.x;", "mov.u32 %r1, %tid.y;", "mov.u32 %r1, %tid.z;", "mov.u32 %r1, %tid.w;", "mov.u32 %r1, %tid.q;"],
        # %envreg names raise an error, other names of the same length do not
        ["mov.b32 %r1, %envreg3;", "mov.b32 %r1, %envrex3;", "mov.b32 %r1, %envreg12;", "mov.b32 %r1, %envreg33;", "mov.b32 %r1, %envreg0;"],
        # predicates, labels, branches, blocks
        ["@%p1 bra L1;", "@!%p1 bra L1;", "@%p22 bra LONGER_LABEL;", "L1:", "LONGER_LABEL:", "bra.uni L1;", "{", "}", "ret;"],
        # variables
        [".reg .b32 %r<10>;", ".reg .b32 %r<11>;", ".reg .b32 %q<10>;", ".reg .pred %p;", ".reg .f32 %a, %b;", ".local .align 8 .b8 buf[16];",
         ".local .align 8 .b8 buf[32];", ".shared .u32 s = 1;"],
        # .loc lines ride with the next statement; the extended forms read identifier spellings
        [".loc 1 2 3", ".loc 1 2 4", ".loc 1 2 3, function_name foo, inlined_at 1 2 3", ".loc 1 2 3, function_nam foo, inlined_at 1 2 3"],
        # calls reserve an error slot and need the function table: never templated
        ["call foo, (%r1);", "call (%r1), foo, (%r2);", "call bar;"],
        # vectors, strings, pragmas
        ["ld.global.v4.u32 {%r1,%r2,%r3,%r4}, [%rd1];", "ld.global.v4.u32 {%r1, %r2, %r3, _}, [%rd1];", "ld.global.v2.u32 {%r1,%r2}, [%rd1];",
         ".pragma \"nounroll\";", ".pragma \"unroll 4\";"],
        # errors inside one statement of a shape that is fine elsewhere
        ["add.s32 %r1, %r2;", "add.s32 %r1, %r2, %r3, %r4;", "add.s33 %r1, %r2, %r3;", "add.s32 %r1, %r2, %r3"],
    ]
    out = []
    for g in groups:
        stmts = []
        for rep in range(3):
            stmts += g
        out.append(body("\n".join(stmts)))
    # everything together, twice, in two functions: classes are shared across functions and modules
    allstmts = "\n".join(st for g in groups[:7] for st in g)
    out.append(body(allstmts + "\n" + allstmts))
    return out


def bulk_cases(n=9000):
    """Arrays whose initialiser is long enough for the bulk path (one thread per element), regular and not."""
    import random
    rng = random.Random(5)

    def elems(k):
        out = []
        for _ in range(k):
            r = rng.random()
            out.append(str(rng.randrange(1 << 31)) if r < 0.5 else hex(rng.randrange(1 << 32)) if r < 0.8 else "-%d" % rng.randrange(1000))
        return out

    def mod(decl, items, tail="};"):
        return HEADER + decl + " = {" + ", ".join(items) + tail + "\n.visible .entry k()\n{\nret;\n}\n"

    e = elems(n)
    f = ["%d.5" % i for i in range(n)]
    names = ["sym%d" % (i % 7) for i in range(n)]
    out = [
        mod(".global .align 4 .s64 a[%d]" % n, e),                               # regular
        mod(".global .align 4 .s64 a[%d]" % (n + 100), e),                       # fewer elements than the dimension
        mod(".global .align 4 .s64 a[%d]" % (n - 1), e),                         # one element too many
        mod(".const .align 8 .f64 c[%d]" % n, f),                                # floats
        mod(".global .align 8 .u64 p[%d]" % n, names),                           # names
        mod(".global .align 4 .s64 a[%d]" % n, e[:-1] + ["99999999999999999999999"]),   # an element that overflows
        mod(".global .align 4 .s64 a[%d]" % n, e, tail=",};"),                   # trailing comma
        mod(".global .align 4 .s64 a[%d]" % n, e[:50] + ["{1}"] + e[51:]),       # a brace inside
        mod(".global .align 4 .s64 a[%d]" % n, e[:50] + [""] + e[51:]),          # an empty element
        mod(".global .align 4 .s64 a[%d]" % n, e, tail="}"),                     # no semicolon
        mod(".global .align 4 .s64 a[%d]" % n, e[:70] + ["1 2"] + e[71:]),       # two numbers without a comma
        mod(".global .align 4 .s64 a[]" , e),                                    # unsized array
        mod(".global .align 4 .v2 .s64 a[%d]" % n, e),                           # vector type: no initialiser list allowed
        mod(".extern .global .align 4 .s64 a[%d]" % n, e),
    ]
    # two long arrays and ordinary code in one module
    out.append(HEADER + ".global .align 4 .s64 a[%d] = {%s};\n.global .align 4 .u32 b[%d] = {%s};\n" % (n, ", ".join(e), n, ", ".join(e[::-1]))
               + ".visible .entry k()\n{\n" + DECLS + "\nadd.s32 %r1, %r2, %r3;\nret;\n}\n")
    return out


def capacity_cases():
    """More distinct statement classes than the class store holds, and names at the length limits of the packed forms."""
    # 270,000 classes: the text of a string is part of its statement's class; and as many immediates, which are one class
    many = "\n".join(".pragma \"n%d\";\nmov.u32 %%r1, %d;" % (i, i) for i in range(270000))
    out = [body(many)]
    longs = []
    for n in (125, 126, 127, 128, 254, 255, 256, 300, 65534, 65535, 65536, 70000):
        for ch in "ab":
            longs.append("add.s32 %%r1, %%%s, %%r3;" % (ch * n))
            longs.append("L%s: bra L%s;" % (ch * n, ch * n))
    out.append(body("\n".join(longs)))
    # more units without a template than the "few" threshold of the decode stage: calls are never templated
    calls = "\n".join(("call foo, (%%r%d);" % (i % 9)) if i % 3 else "call.uni bar;" for i in range(140000))
    out.append(HEADER + ".func foo(.param .b32 p)\n{\nret;\n}\n.visible .entry k()\n{\n" + DECLS + "\n" + calls + "\nret;\n}\n")
    return out


def nested_damage_cases():
    """A stray token in front of a '}' below d levels of nested blocks.  The reference recovers a failed block from its
    '{' and parses its contents again as statements of the enclosing block, at every level: 2^d times the work and as
    many appended errors.  Shallow damage must come out identical (errors repeated as the reference repeats them); deep
    damage must end with the verdict ReferenceDiverges on both sides, after the same number of statement attempts."""
    out = []
    for depth in (1, 2, 3, 5, 8, 12, 16, 28, 32):
        lines = []
        for d in range(depth):
            lines.append("\t" * d + "{")
            lines.append("\t" * (d + 1) + ".reg .b32 %%t%d;" % d)
            lines.append("\t" * (d + 1) + "add.s32 %r1, %r2, %r3;")
        lines.append("\t" * depth + ".bar")
        for d in reversed(range(depth)):
            lines.append("\t" * d + "}")
        out.append(body("\n".join(lines)))
        out.append(body("\n".join(lines)) + ".global .u32 after;\n.visible .entry k2()\n{\nret;\n}\n")
    return out


def confined_damage_cases(n_funcs=12, n_instr=60):
    """Modules of several functions that call one another, damaged in one place: everything in front of the damaged
    top-level directive must keep its speculated units, only the tail goes through the sequential parser (some of the
    damage is recovered inside its statement and needs no sequential parse at all).  Returns (text, fraction of the
    text in front of the damaged directive) pairs."""
    def func(i, extra=""):
        lines = [".func (.param .b32 r) f%d(.param .b32 a)" % i, "{", ".reg .b32 %r<8>;", ".reg .pred %p<2>;", ".param .b32 pa;", ".param .b32 pr;"]
        for k in range(n_instr):
            lines.append("add.s32 %%r%d, %%r%d, %d;" % (k % 7 + 1, (k + 1) % 7 + 1, k))
            if k % 17 == 5 and i > 0:
                # a call of an earlier function (declared in front of the damage or behind it) and of an unknown one
                lines.append("st.param.b32 [pa], %r1;")
                lines.append("call (pr), f%d, (pa);" % (i // 2))
                lines.append("call (pr), nowhere%d, (pa);" % i)
            if k == n_instr // 2:
                lines.append(extra)
        lines += ["ret;", "}"]
        return "\n".join(l for l in lines if l)
    out = []
    for damage in ("{", "(", ".reg .b32 %dup<2>; { add.s32 %r1, %r2, %r3;", "}", "} }", "foo bar {"):
        for where in (0, n_funcs // 2, n_funcs - 1):
            funcs = [func(i, damage if i == where else "") for i in range(n_funcs)]
            text = HEADER + "\n".join(funcs) + "\n.global .u32 after;\n"
            front = len(HEADER + "\n".join(funcs[:where]))
            out.append((text, front / len(text)))
    # a module cut off in the middle of its last function
    funcs = [func(i) for i in range(n_funcs)]
    text = HEADER + "\n".join(funcs)
    cut = len(text) - len(funcs[-1]) // 2
    out.append((text[:cut], len(HEADER + "\n".join(funcs[:-1])) / cut))
    return out


STRAY_TOKENS = ["}", "(", ")", "foo", "foo bar baz;", ":", ",", ".entry", ".global", "12345", "mov.v2.u32 {%r1, %r2, %r3;"]


def stray_token_modules(text, at_fraction=0.5):
    """`text` (bytes) with one stray token on a line of its own at a line start near the given fraction: damage that
    the speculated units recover from without the sequential parser ('{' is not among them: an unclosed scope changes
    what everything behind it means, in the reference as well)."""
    at = text.find(b"\n", int(at_fraction * len(text))) + 1
    return [text[:at] + tok.encode() + b"\n" + text[at:] for tok in STRAY_TOKENS]


def negative_decimal_side_file(n=1000):
    """Module-level scalars initialised with NEGATIVE decimal floats and integers: the reference has no rule for '-' in
    front of a float literal (ptx_parser/src/lib.rs:366-377), so every float directive must be rejected the same way,
    while negative integers are fine."""
    import random
    rng = random.Random(9)
    lines = []
    for i in range(n):
        r = rng.random()
        if r < 0.4:
            lines.append(".global .f64 c%d = -%.17g;" % (i, rng.random() * 1e6))
        elif r < 0.7:
            lines.append(".global .f32 c%d = -%.9g;" % (i, rng.random() * 100))
        elif r < 0.85:
            lines.append(".global .s32 c%d = -%d;" % (i, rng.randrange(1 << 31)))
        else:
            lines.append(".global .f64 c%d = %.17g;" % (i, rng.random()))
    return HEADER + "\n".join(lines) + "\n.visible .entry k()\n{\nret;\n}\n"


def dense_token_texts():
    """Texts with more tokens per 8 KiB lexer tile than the emit step lists at a time (3,072), and tiles whose tokens are
    nearly all numbers or nearly all keyword candidates (more than the 2,048 either list of a pass holds)."""
    import random
    rng = random.Random(11)
    texts = ["1," * 20000, ";" * 30000, "12 " * 12000, "ab " * 12000, "add mov " * 6000, ".f32.u8 " * 5000, "0x1F 1.5 " * 5000,
             "{%r1,%r2}," * 4000, "a+1," * 9000]
    pieces = [",", ";", "1", "a", ".x", "%r", "+", "-", "[", "]", "0f3F800000", "ld", "st", " ", "\n", "12U", ".5", "::", "@!p"]
    for _ in range(6):
        texts.append("".join(rng.choice(pieces) for _ in range(30000)))
    return texts


def numbers_across_tile_ends():
    """One module per probe and shift: a `mov` whose immediate is the probe, placed so that the probe slides across the
    end of the first 8 KiB lexer tile (the module has to begin where a tile begins: parse it alone)."""
    probes = ["123456789.12345678e-05", "1.5e+3", "1.5e", "7.25", "0d3FF0000000000000", "0f3F800000", "0f3F80000", "0x1F2e3D4cU", "4294967295U",
              "18446744073709551615", "18446744073709551616", "017", "09", "0", "5", "123456789", "1234567890", "2147483648", "999999999U",
              "0f3F80000G", "0F3f80000a", "12.", "00", "0x", "0d1"]
    head = HEADER + ".visible .entry k()\n{\n.reg .f64 %fd<4>;\n"
    texts = []
    for probe in probes:
        for shift in range(0, 24):
            stmt = "mov.f64 %%fd1, %s;\n" % probe
            # filler statements up to the tile end, then the probe shifted across it
            target = 8192 - len("mov.f64 %fd1, ") - len(probe) + shift
            body, filler = "", "add.s32 %r1, %r2, 3;\n"
            while len(head) + len(body) + len(filler) < target - 40:
                body += filler
            pad = target - len(head) - len(body)
            body += "/*" + "x" * max(0, pad - 5) + "*/\n" if pad >= 5 else " " * max(0, pad)
            texts.append(head + body + stmt + "ret;\n}\n")
    return texts
