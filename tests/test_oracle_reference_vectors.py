"""Pins the CPU oracle against the vectors that the reference's own tests hold for the PTX front end.

Sources (paths inside the reference project):
  * inline parser tests                      ptx_parser/src/lib.rs:4529-4898
  * every .ptx fixture its tests parse       ptx/src/test/**, ptx/src/pass/test/**, zluda/src/impl/test_ptx/**
    (all enter through parse_module_checked(..).unwrap(), ptx/src/test/mod.rs:32-43)
  * literal rules restated from              ptx_parser/src/lib.rs:222-377 and the token regexes at lib.rs:1944-1979
The fixture files are read from a reference checkout when one is mounted; they are not copied into this repository.
"""
import glob
import os

import pytest

from oracle_lib import CHECKED, ERRORS_ONLY, UNCHECKED

import reference_fixtures

HEADER = ".version 6.5\n.target sm_30\n.address_size 64\n"


def body(stmts, decls=".reg .b32 %r<10>; .reg .b64 %rd<10>; .reg .f32 %f<10>; .reg .f64 %fd<4>; .reg .pred %p<4>;"):
    return HEADER + ".visible .entry k()\n{\n" + decls + "\n" + stmts + "\nret;\n}\n"


def instr_line(oracle, stmt):
    st, dump = oracle.parse(body(stmt))
    assert st == 0, dump
    lines = [l.strip() for l in dump.split("\n") if l.strip().startswith("Instruction(")]
    return lines[0]


# ------------------------------------------------------------------ header forms (lib.rs:4529-4575, ptx/src/test/mod.rs:45-48)
@pytest.mark.parametrize("target,sm", [("sm_11", 11), ("sm_90a", 90), ("sm_30", 30)])
def test_target_forms(oracle, target, sm):
    st, dump = oracle.parse(".version 6.5\n.target %s\n" % target)
    assert st == 0
    assert "sm_version: %d," % sm in dump


def test_target_two_letter_suffix_rejected(oracle):
    st, dump = oracle.parse(".version 6.5\n.target sm_90ab\n")
    assert st == 1 and "Parser(ContextError)" in dump


def test_version_target_debug_no_body(oracle):
    st, dump = oracle.parse(".version 6.5 .target sm_30, debug")
    assert st == 0
    assert "ptx_version: (6, 5), sm_version: 30, address_size: 32, invalid_directives: 0, directives: 0" in dump


# ------------------------------------------------------------------ recovery text and extent (lib.rs:4577-4692)
def test_report_unknown_instruction(oracle):
    text = """
            .version 6.5
            .target sm_30
            .address_size 64

            .visible .entry add(
                .param .u64 input,
                .param .u64 output
            )
            {
                .reg .u64 	    in_addr;
                .reg .u64 	    out_addr;
                .reg .u64 	    temp;
                .reg .u64 	    temp2;

                ld.param.u64 	in_addr, [input];
                ld.param.u64 	out_addr, [output];

                ld.u64          temp, [in_addr];
                unknown_op1.asdf foobar;
                add.u64		    temp2, temp, 1;
                unknown_op2 temp2, temp;
                st.u64          [out_addr], temp2;
                ret;
            }"""
    assert oracle.errors(text) == [
        'UnrecognizedStatement("unknown_op1.asdf foobar;")',
        'UnrecognizedStatement("unknown_op2 temp2, temp;")',
    ]


def test_report_unknown_instruction_with_braces(oracle):
    text = HEADER + ".visible .entry unrecognized_braces(\n)\n{\n mov.u32 foo, {} {};\n ret;\n}"
    assert oracle.errors(text) == ['UnrecognizedStatement("mov.u32 foo, {} {};")']


def test_report_unknown_directive(oracle):
    text = HEADER + """
            .broken_directive_fail; 34; {

            .visible .entry add(
                .param .u64 input,
                .param .u64 output
            )
            {
                .reg .u64 	    in_addr;
                ld.param.u64 	in_addr, [input];
                ret;
            }

            section foobar }"""
    assert oracle.errors(text) == [
        'UnrecognizedDirective(".broken_directive_fail; 34; {")',
        'UnrecognizedDirective("section foobar }")',
    ]


def test_report_unknown_type_in_directive(oracle):
    text = ".version 4.1\n.target sm_52\n.address_size 64\n.global .bad_type foo;\n.const .b32 bar;\n"
    assert oracle.errors(text) == ['UnrecognizedDirective(".global .bad_type foo;")']


def test_invalid_directive_count(oracle):
    text = HEADER + """
            .global .b32 global[4] = {  unknown (1),   2,   3,   4};
            .visible .entry func1()
            {
                st.u64          [out_addr], temp2;
                ret;
            }
            .visible .entry func1()
            {
                broken_instruction;
                ret;
            }"""
    st, dump = oracle.parse(text, UNCHECKED)
    assert "invalid_directives: 2, directives: 1" in dump


def test_file_directive_is_ignored_silently(oracle):
    text = HEADER + '.file 1 "example.cu"\n.visible .entry func1()\n{\n ret;\n}'
    st, dump = oracle.parse(text)
    assert st == 0 and "invalid_directives: 0, directives: 1" in dump


def test_extern_func_noreturn(oracle):
    text = ".version 6.4\n.target sm_70\n.address_size 64\n\n.extern .func __assertfail() .noreturn;\n"
    st, dump = oracle.parse(text)
    assert st == 0 and "tuning: [NoReturn], body: None" in dump


def test_dwarf_section_body(oracle):
    lines = "\n".join(".b8 %d   // comment" % (i % 90) for i in range(55))
    text = HEADER + ".section .debug_abbrev\n{\n" + lines + "\n}\n"
    st, dump = oracle.parse(text)
    assert st == 0 and "errors: 0" in dump


# ------------------------------------------------------------------ zero padding (lib.rs:4850-4898)
def test_const_zero_pad(oracle):
    st, dump = oracle.parse(HEADER + ".const .align 4 .b8 constData[8];")
    assert st == 0
    assert "array_init: [" + ", ".join(["Imm(U64(0))"] * 8) + "]" in dump
    assert "align: Some(4), v_type: Array(None, B8, [8])" in dump


def test_global_zero_init(oracle):
    st, dump = oracle.parse(HEADER + ".global .align 4 .b8 constData;")
    assert st == 0 and "v_type: Scalar(B8), state_space: Global, array_init: [Imm(U64(0))]" in dump


def test_partial_initializer_is_padded_with_typed_zero(oracle):
    st, dump = oracle.parse(HEADER + ".global .s32 x[4] = {1};\n.global .f32 y[2] = {0f3F800000};")
    assert "array_init: [Imm(S64(1)), Imm(S64(0)), Imm(S64(0)), Imm(S64(0))]" in dump
    assert "array_init: [Imm(F32(bits=0x3F800000)), Imm(F64(bits=0x0000000000000000))]" in dump


# ------------------------------------------------------------------ literal conversion (lib.rs:222-377)
LITERALS = [
    ("10", "Imm(S64(10))", None),
    ("18446744073709551615", "Imm(U64(18446744073709551615))", None),
    ("18446744073709551616", "Imm(U64(0))", "ParseInt(PosOverflow)"),
    ("10U", "Imm(U64(10))", None),
    ("-10U", "Imm(S64(-10))", None),
    ("-9223372036854775808", "Imm(S64(-9223372036854775808))", None),
    ("-9223372036854775809", "Imm(S64(0))", "ParseInt(NegOverflow)"),
    ("010", "Imm(S64(8))", None),
    ("09", "Imm(U64(0))", "ParseInt(InvalidDigit)"),
    ("0", "Imm(S64(0))", None),
    ("0x1F", "Imm(S64(31))", None),
    ("0X1f", "Imm(S64(31))", None),
    ("0xFFFFFFFFFFFFFFFF", "Imm(U64(18446744073709551615))", None),
    ("0xFFU", "Imm(U64(255))", None),
    ("0xU", "Imm(U64(0))", "ParseInt(Empty)"),
    ("0xZZ", "Imm(U64(0))", "ParseInt(InvalidDigit)"),
    ("0f3F800000", "Imm(F32(bits=0x3F800000))", None),
    ("0fGGGGGGGG", "Imm(F32(bits=0x00000000))", "ParseInt(InvalidDigit)"),
    ("0d3FF0000000000000", "Imm(F64(bits=0x3FF0000000000000))", None),
    ("1.5", "Imm(F64(bits=0x3FF8000000000000))", None),
    (".5", "Imm(F64(bits=0x3FE0000000000000))", None),
    ("1.5e-3", "Imm(F64(bits=0x3F589374BC6A7EFA))", None),
    ("0.1", "Imm(F64(bits=0x3FB999999999999A))", None),
    ("1.7976931348623157e308", "Imm(F64(bits=0x7FEFFFFFFFFFFFFF))", None),
    ("4.9e-324", "Imm(F64(bits=0x0000000000000001))", None),
    ("1.0e400", "Imm(F64(bits=0x7FF0000000000000))", None),
    ("WARP_SZ", "Imm(U64(32))", None),
]


@pytest.mark.parametrize("lit,expect,err", LITERALS)
def test_literal(oracle, lit, expect, err):
    text = body("mov.b64 %rd1, " + lit + ";")
    dump = oracle.parse(text, UNCHECKED)[1]
    if err is None:
        assert "src: " + expect in dump
    else:
        # a directive that raised an error is dropped (lib.rs:613-615), so only the error is visible
        assert "invalid_directives: 1, directives: 0" in dump
    assert oracle.errors(text) == ([err] if err else [])


@pytest.mark.parametrize("stmt", [
    "mov.f64 %fd1, -1.5;", "mov.f32 %f1, -0f3F800000;", "mov.f32 %f1, 0f3F8000;", "mov.f64 %fd1, 2.E5;",
    "mov.f64 %fd1, 2.;", "bra add;", ".reg .b32 %z<0>;", ".reg .b32 %a, %b<4>;", "ld.u32.v2 {%r1,%r2}, [%rd1];",
    "add.s32.s32 %r1, %r2, %r3;", "shf.l.wrap.b32 %r1, %r2.r, %r3, %r4;",
])
def test_rejected_statements(oracle, stmt):
    errs = oracle.errors(body(stmt))
    assert len(errs) >= 1 and errs[-1].startswith("UnrecognizedStatement("), errs


def test_operand_forms(oracle):
    line = instr_line(oracle, "ld.global.u32 %r1, [%rd1+-16];")
    assert 'src: RegOffset("%rd1", -16)' in line
    text = body("ld.global.u32 %r1, [%rd1+2147483648];")
    assert oracle.errors(text) == ["ParseInt(PosOverflow)"]
    assert 'VecMember("%v", 0)' in oracle.parse(body("mov.u32 %r1, %v.x;"), UNCHECKED)[1]
    assert oracle.errors(body("mov.u32 %r1, %v.q;")) == ["WrongVectorElement"]
    line = instr_line(oracle, "mov.b64 %rd1, {%r1, 7};")
    assert 'src: VecPack([Reg("%r1"), Imm(S64(7))])' in line


def test_label_named_like_opcode(oracle):
    st, dump = oracle.parse(body("add:\n"))
    assert st == 0 and 'Label("add")' in dump


def test_address_size_16_is_an_unrecognized_directive(oracle):
    text = ".version 6.5\n.target sm_30\n.address_size 16\n.visible .entry k() { ret; }"
    dump = oracle.parse(text, UNCHECKED)[1]
    assert "address_size: 32, invalid_directives: 1" in dump
    assert any(e.startswith("UnrecognizedDirective(") for e in oracle.errors(text))


def test_register_count_overflow_leaves_both_errors(oracle):
    errs = oracle.errors(body(".reg .b32 %q<99999999999>;"))
    assert errs == ["ParseInt(PosOverflow)", 'UnrecognizedStatement(".reg .b32 %q<99999999999>;")']


def test_lex_errors(oracle):
    for bad in ["#", "&", "~", "/* never closed", "\"open string"]:
        st, dump = oracle.parse(HEADER + bad)
        assert st == 1 and "Lexer(" in dump
        # a lex error returns before parsing: only Lexer errors are listed
        assert all(e.startswith("Lexer(") for e in oracle.errors(HEADER + bad))
    # parse_for_errors keeps going after a lex error (lib.rs:392-426)
    errs = oracle.errors(HEADER + ".visible .entry k() { # ret; }", ERRORS_ONLY)
    assert errs[0].startswith("Lexer(") and len(errs) == 1


def test_call_resolution(oracle):
    text = HEADER + """
.func (.reg .b32 r) f(.reg .b32 a, .reg .b32 b);
.visible .entry k()
{
 .reg .b32 %r<4>;
 call (%r1), f, (%r2, %r3);
 call (%r1), f, (%r2);
 call g;
 call.uni k;
 ret;
}
"""
    dump = oracle.parse(text, UNCHECKED)[1]
    assert oracle.errors(text, UNCHECKED) == ["MalformedCall", "UnknownFunction", "UnknownFunction"]
    # the directive that raised the errors is dropped
    assert "invalid_directives: 1, directives: 1" in dump


def test_semantic_errors_keep_the_instruction(oracle):
    assert oracle.errors(body("cvt.f32.u32 %f1, %r1;")) == ['SyntaxError("missing rounding mode for cvt")']
    assert oracle.errors(body("setp.lt.ftz.u32 %p1, %r1, %r2;")) == ["NonF32Ftz"]
    assert oracle.errors(body("setp.ltu.u32 %p1, %r1, %r2;")) == ["WrongType"]
    line = instr_line(oracle, "add.f32.rn %f1, %f2, %f3;")
    assert "rounding: NearestEven" in line and "is_fusable: false" in line


def test_lexer_longest_match(oracle):
    def kinds(s):
        return [oracle.token_text(k) or {5: "IDENT", 6: "DOTIDENT", 18: "F32HEX", 19: "F64HEX", 20: "HEX", 21: "F64",
                                          22: "DECIMAL", 7: "STRING"}[k] for k, _, _ in oracle.lex(s)[0]]
    assert kinds("address add .f32x .f32") == ["IDENT", "add", "DOTIDENT", ".f32"]
    assert kinds(".shared::cta .shared::ctax .L2::64B .L2::x") == [
        ".shared::cta", ".shared::cta", "IDENT", ".L2::64B", ".L2", ":", ":", "IDENT"]
    assert kinds(".1d .1 1.5e-3 1.5e 0f3F8000 0f3F800000 123abc 10U") == [
        ".1d", "F64", "F64", "F64", "IDENT", "DECIMAL", "IDENT", "F32HEX", "DECIMAL", "IDENT", "DECIMAL"]
    assert kinds("a/*x*/b//c\nd \"s//\" /**/") == ["IDENT", "IDENT", "IDENT", "STRING"]


# ------------------------------------------------------------------ the reference's accept corpus
def test_every_reference_fixture_is_accepted(oracle):
    """Every `ptx` test of the reference feeds its input to parse_module_checked(..).unwrap() (ptx/src/test/mod.rs:32-75;
    the pass tests parse the part before their output marker, ptx/src/pass/test/mod.rs:14-36).  spirv_fail/ and
    spirv_build/ are not referenced by any reference test."""
    import hashlib
    rows = reference_fixtures.rows()
    assert len(rows) >= 240
    for r in rows:
        text = r["text"].encode("latin-1")
        st, dump = oracle.parse(text, CHECKED)
        if "spirv_fail" not in r["name"] and "spirv_build" not in r["name"]:
            assert st == 0, (r["name"], dump[-600:])
        assert (st == 0) == r["accepted"], r["name"]
        assert hashlib.sha256(dump.encode()).hexdigest() == r["sha256"][0], r["name"]
    assert oracle.schema_ok()


def test_reference_fixture_values(oracle):
    """Spot values that the reference's LLVM goldens depend on (ptx/src/test/ll/*.ll)."""
    texts = reference_fixtures.texts()

    def dump_of(name):
        return oracle.parse(texts["ptx/src/test/spirv_run/" + name])[1]
    assert "Imm(S64(-" in dump_of("constant_negative.ptx")
    assert "Imm(F32(bits=0x" in dump_of("constant_f32.ptx")
    d = dump_of("global_array_f32.ptx")
    assert "Array(None, F32, [" in d and "Imm(F32(bits=0x" in d
    assert "CreatePolicyFractional" in dump_of("createpolicy.ptx")
    assert 'VecMember("%ntid", 0)' in oracle.parse(texts["ptx/src/test/operands.ptx"])[1]
