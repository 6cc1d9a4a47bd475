#!/usr/bin/env python3
"""Generate ptx_lex_tables.h: byte classes and the transition table of the lockstep token automaton.

The automaton restates the token rules of ptx_parser's logos lexer (ptx_parser/src/lib.rs:1930-2030) as one
byte-at-a-time machine so that every GPU thread of a warp executes the same loop body:

  * skip rule: whitespace, // comments, /* */ comments
  * Ident / DotIdent, String, Hex, F32Hex (exactly 8 alnum), F64Hex (exactly 16), F64 with optional exponent,
    Decimal with optional U, the single-character tokens
  * longest match with back-up: where a longer token could still follow (exponent, 0x, 0f, 0d, "1.") the machine
    remembers the last accepted end and returns to it when the longer form fails
Keywords are not decided here: identifiers and dot-identifiers are classified afterwards by a hash lookup, and the
"::" literals (.shared::cta ...) are checked by a helper when a dot-identifier is followed by ':'.

Usage: gen_lex_tables.py --out DIR [--out DIR2]
"""
import argparse
import os

# ---- byte classes
CLASSES = ["WS", "NL", "LETTER", "E", "X", "F", "D", "U", "ZERO", "D123", "DIGIT", "USCORE", "PERCENT", "DOT", "COLON",
           "SIGN", "SLASH", "STAR", "QUOTE", "HARD", "OTHER"]
C = {n: i for i, n in enumerate(CLASSES)}


def byte_class(b):
    ch = chr(b)
    if ch in " \t\v\f":
        return C["WS"]
    if ch in "\n\r":
        return C["NL"]
    if ch in "eE":
        return C["E"]
    if ch in "xX":
        return C["X"]
    if ch in "fF":
        return C["F"]
    if ch in "dD":
        return C["D"]
    if ch == "U":
        return C["U"]
    if ch.isascii() and ch.isalpha():
        return C["LETTER"]
    if ch == "0":
        return C["ZERO"]
    if ch in "123":
        return C["D123"]
    if ch in "456789":
        return C["DIGIT"]
    if ch in "_$":
        return C["USCORE"]
    if ch == "%":
        return C["PERCENT"]
    if ch == ".":
        return C["DOT"]
    if ch == ":":
        return C["COLON"]
    if ch in "+-":
        return C["SIGN"]
    if ch == "/":
        return C["SLASH"]
    if ch == "*":
        return C["STAR"]
    if ch == '"':
        return C["QUOTE"]
    if ch in ",;@|!()[]{}<>=":
        return C["HARD"]
    return C["OTHER"]


ALPHA = ["LETTER", "E", "X", "F", "D", "U"]
DIGITS = ["ZERO", "D123", "DIGIT"]
IDENTC = ALPHA + DIGITS + ["USCORE"]
ALNUM = ALPHA + DIGITS

# ---- states
STATES = ["S0", "IDENT", "SIGIL1", "DOT1", "DOTSIG1", "DOTIDENT", "FRACDIM", "FRAC", "EXP_E", "EXP_SIGN", "EXP_D", "DEC",
          "DECDOT", "ZERO", "HEX0", "HEX", "HFLOAT", "SLASH1", "LINE", "BLOCK", "STAR", "STR", "SLASH_IN"]
S = {n: i for i, n in enumerate(STATES)}

# ---- actions
ACTIONS = ["NONE", "BEGIN", "SINGLE", "END", "END_INCL", "ACCEPT", "BACKUP", "ERR_HERE", "ERR_TOKEN", "COUNT",
           "BEGIN_HF32", "BEGIN_HF64", "COLON_CHECK", "REWIND_DOT", "ERR_SLASH", "DIM"]
A = {n: i for i, n in enumerate(ACTIONS)}
# token kind produced by END / END_INCL in a state (names of PtxTok members)
END_KIND = {"IDENT": "T_IDENT", "DOTIDENT": "T_DOTIDENT", "DOT1": "T_DOT", "FRACDIM": "T_F64", "FRAC": "T_F64", "EXP_D": "T_F64",
            "DEC": "T_DECIMAL", "ZERO": "T_DECIMAL", "HEX": "T_HEX", "STR": "T_STRING", "DECDOT": "T_DECIMAL", "HEX0": "T_DECIMAL",
            "HFLOAT": "T_DECIMAL", "EXP_E": "T_F64", "EXP_SIGN": "T_F64"}


def build():
    n_s, n_c = len(STATES), len(CLASSES)
    T = [[None] * n_c for _ in range(n_s)]

    def setc(state, classes, nxt, act):
        for c in classes:
            T[S[state]][C[c]] = (S[nxt], A[act])

    def default(state, nxt, act):
        for c in range(n_c):
            if T[S[state]][c] is None:
                T[S[state]][c] = (S[nxt], A[act])

    # S0: between tokens, in code
    setc("S0", ["WS", "NL"], "S0", "NONE")
    setc("S0", ALPHA, "IDENT", "BEGIN")
    setc("S0", ["USCORE", "PERCENT"], "SIGIL1", "BEGIN")
    setc("S0", ["ZERO"], "ZERO", "BEGIN")
    setc("S0", ["D123", "DIGIT"], "DEC", "BEGIN")
    setc("S0", ["DOT"], "DOT1", "BEGIN")
    setc("S0", ["COLON", "SIGN", "HARD"], "S0", "SINGLE")
    setc("S0", ["SLASH"], "SLASH1", "BEGIN")
    setc("S0", ["QUOTE"], "STR", "BEGIN")
    setc("S0", ["STAR", "OTHER"], "S0", "ERR_HERE")
    # identifiers
    setc("IDENT", IDENTC, "IDENT", "NONE")
    default("IDENT", "S0", "END")
    setc("SIGIL1", IDENTC, "IDENT", "NONE")
    default("SIGIL1", "S0", "ERR_TOKEN")          # a lone _ $ % : one-byte error, the current byte is looked at again
    # '.'
    setc("DOT1", ALPHA, "DOTIDENT", "NONE")
    setc("DOT1", ["USCORE", "PERCENT"], "DOTSIG1", "NONE")
    setc("DOT1", ["D123"], "FRACDIM", "NONE")
    setc("DOT1", ["ZERO", "DIGIT"], "FRAC", "NONE")
    default("DOT1", "S0", "END")
    setc("DOTSIG1", IDENTC, "DOTIDENT", "NONE")
    default("DOTSIG1", "S0", "REWIND_DOT")         # "." is a token by itself; continue with the sigil byte
    setc("DOTIDENT", IDENTC, "DOTIDENT", "NONE")
    setc("DOTIDENT", ["COLON"], "S0", "COLON_CHECK")
    default("DOTIDENT", "S0", "END")
    # fractions and exponents
    setc("FRACDIM", ["D"], "S0", "DIM")            # ".1d" ".2d" ".3d" ('D' is told apart in the action)
    setc("FRACDIM", DIGITS, "FRAC", "NONE")
    setc("FRACDIM", ["E"], "EXP_E", "ACCEPT")
    default("FRACDIM", "S0", "END")
    setc("FRAC", DIGITS, "FRAC", "NONE")
    setc("FRAC", ["E"], "EXP_E", "ACCEPT")
    default("FRAC", "S0", "END")
    setc("EXP_E", ["SIGN"], "EXP_SIGN", "NONE")
    setc("EXP_E", DIGITS, "EXP_D", "NONE")
    default("EXP_E", "S0", "BACKUP")
    setc("EXP_SIGN", DIGITS, "EXP_D", "NONE")
    default("EXP_SIGN", "S0", "BACKUP")
    setc("EXP_D", DIGITS, "EXP_D", "NONE")
    default("EXP_D", "S0", "END")
    # integers
    setc("DEC", DIGITS, "DEC", "NONE")
    setc("DEC", ["U"], "S0", "END_INCL")
    setc("DEC", ["DOT"], "DECDOT", "ACCEPT")
    default("DEC", "S0", "END")
    setc("DECDOT", DIGITS, "FRAC", "NONE")
    default("DECDOT", "S0", "BACKUP")
    setc("ZERO", ["X"], "HEX0", "ACCEPT")
    setc("ZERO", ["F"], "HFLOAT", "BEGIN_HF32")
    setc("ZERO", ["D"], "HFLOAT", "BEGIN_HF64")
    setc("ZERO", DIGITS, "DEC", "NONE")
    setc("ZERO", ["U"], "S0", "END_INCL")
    setc("ZERO", ["DOT"], "DECDOT", "ACCEPT")
    default("ZERO", "S0", "END")
    setc("HEX0", ALNUM, "HEX", "NONE")
    default("HEX0", "S0", "BACKUP")
    setc("HEX", ALNUM, "HEX", "NONE")
    default("HEX", "S0", "END")
    setc("HFLOAT", ALNUM, "HFLOAT", "COUNT")       # ends itself when the digit count is reached
    default("HFLOAT", "S0", "BACKUP")
    # comments and strings
    setc("SLASH1", ["SLASH"], "LINE", "NONE")
    setc("SLASH1", ["STAR"], "BLOCK", "NONE")
    default("SLASH1", "S0", "ERR_SLASH")           # a lone '/': one-byte error, look at the current byte again
    setc("SLASH_IN", ["SLASH"], "LINE", "NONE")    # chunk starts right after a '/' that another thread owns
    setc("SLASH_IN", ["STAR"], "BLOCK", "NONE")
    default("SLASH_IN", "S0", "BACKUP")            # (BACKUP with nothing accepted: just look at the byte again)
    setc("LINE", ["NL"], "S0", "NONE")
    default("LINE", "LINE", "NONE")
    setc("BLOCK", ["STAR"], "STAR", "NONE")
    default("BLOCK", "BLOCK", "NONE")
    setc("STAR", ["SLASH"], "S0", "NONE")
    setc("STAR", ["STAR"], "STAR", "NONE")
    default("STAR", "BLOCK", "NONE")
    setc("STR", ["QUOTE"], "S0", "END_INCL")
    default("STR", "STR", "NONE")
    for s in range(n_s):
        for c in range(n_c):
            assert T[s][c] is not None, (STATES[s], CLASSES[c])
    return T


HARD_KIND = {",": "T_COMMA", ";": "T_SEMI", "@": "T_AT", "|": "T_PIPE", "!": "T_EXCL", "(": "T_LPAREN", ")": "T_RPAREN",
             "[": "T_LBRACKET", "]": "T_RBRACKET", "{": "T_LBRACE", "}": "T_RBRACE", "<": "T_LT", ">": "T_GT", "=": "T_EQ",
             ":": "T_COLON", "+": "T_PLUS", "-": "T_MINUS"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", action="append", default=[])
    a = ap.parse_args()
    T = build()
    L = ["// GENERATED by zluda_b200/grammar/gen_lex_tables.py -- do not edit.",
         "// Byte classes and transition table of the lockstep token automaton (see the generator for the rules).",
         "#pragma once", "#include <stdint.h>"]
    L.append("enum { " + ", ".join("LC_%s = %d" % (n, i) for i, n in enumerate(CLASSES)) + ", LC_COUNT = %d };" % len(CLASSES))
    L.append("enum { " + ", ".join("LS_%s = %d" % (n, i) for i, n in enumerate(STATES)) + ", LS_COUNT = %d };" % len(STATES))
    L.append("enum { " + ", ".join("LA_%s = %d" % (n, i) for i, n in enumerate(ACTIONS)) + " };")
    L.append("#define LX_STRIDE 32   // classes per table row")
    L.append("PTX_TABLE uint8_t ptx_lex_class[256] = {")
    for r in range(0, 256, 32):
        L.append("    " + ",".join(str(byte_class(b)) for b in range(r, r + 32)) + ",")
    L.append("};")
    L.append("// entry = next state | action << 8")
    L.append("PTX_TABLE uint16_t ptx_lex_trans[LS_COUNT * LX_STRIDE] = {")
    for s in range(len(STATES)):
        row = [T[s][c][0] | (T[s][c][1] << 8) for c in range(len(CLASSES))] + [0] * (32 - len(CLASSES))
        L.append("    " + ",".join(str(x) for x in row) + ",   // " + STATES[s])
    L.append("};")
    L.append("// token kind that END / END_INCL / BACKUP-from produce in each state")
    L.append("PTX_TABLE uint16_t ptx_lex_end_kind[LS_COUNT] = {" + ", ".join(END_KIND.get(s, "T_ERROR") for s in STATES) + "};")
    # ---- the table the byte loop reads: one 16-bit entry per (state, byte)
    #   bits 0..4   next state
    #   bits 5..8   flags: 1 advance, 2 a token begins here, 4 emit a token, 8 rare action
    #   bits 9..12  with "emit": 1 = the token includes this byte, 2 = the token IS this byte; with "rare": the action
    # The kind of an emitted token is ptx_lex_single[byte] when the token is the byte itself, else
    # ptx_lex_end_kind[state before the byte].
    assert len(STATES) <= 32
    L.append("enum { LF_ADV = 1, LF_BEGIN = 2, LF_EMIT = 4, LF_RARE = 8, LF_INCL = 1, LF_SELF = 2, LF_FLAG_SHIFT = 5, LF_AUX_SHIFT = 9, LF_STATE_MASK = 31 };")
    L.append("PTX_TABLE uint16_t ptx_lex_fused[LS_COUNT * 256] = {")
    for s_i, sname in enumerate(STATES):
        row = []
        for b in range(256):
            nxt, act = T[s_i][byte_class(b)]
            an = ACTIONS[act]
            if an == "NONE":
                e = nxt | (1 << 5)
            elif an == "BEGIN":
                e = nxt | (3 << 5)
            elif an == "END":
                e = nxt | (4 << 5)
            elif an == "END_INCL":
                e = nxt | (5 << 5) | (1 << 9)
            elif an == "SINGLE":
                e = 0 | (5 << 5) | (3 << 9)
            else:
                assert act < 16
                e = nxt | (8 << 5) | (act << 9)
            row.append(str(e))
        L.append("    // " + sname)
        for r in range(0, 256, 32):
            L.append("    " + ",".join(row[r:r + 32]) + ",")
    L.append("};")
    L.append("// kind of the single-character tokens")
    kinds = ["T_ERROR"] * 256
    for ch, k in HARD_KIND.items():
        kinds[ord(ch)] = k
    L.append("PTX_TABLE uint16_t ptx_lex_single[256] = {")
    for r in range(0, 256, 8):
        L.append("    " + ", ".join(kinds[r:r + 8]) + ",")
    L.append("};")
    text = "\n".join(L) + "\n"
    for d in a.out:
        os.makedirs(d, exist_ok=True)
        p = os.path.join(d, "ptx_lex_tables.h")
        if not os.path.exists(p) or open(p).read() != text:
            open(p, "w").write(text)


if __name__ == "__main__":
    main()
