/* Link-time stand-ins for the entry points the reference's command-line front end (src/main.c) references but
 * that are not part of the inference library: trainers, gradient checks, checkpoint inspection, weight saving,
 * dead-code revival and the live viewers (src/ncm.h:233, 265, 324, 351-381,
 * 402-414, 463). With them, the reference's main.c + tok.c + tok_tables.c link against libncm_b200.so and its
 * gen / infer / eval-* / sudoku-stream / gpt2-* / qwen-* commands run on the GPU; a command that needs one of
 * these says so and fails. Parameters are left unspecified on purpose (C11): nothing here reads them.
 *
 *   gcc -O2 -std=c11 -Isrc -c src/main.c src/tok.c src/tok_tables.c
 *   gcc -O2 -std=c11 -c <repo>/saphira-cncm_b200/cli_stubs.c
 *   gcc -o cncm-b200 main.o tok.o tok_tables.o cli_stubs.o -L<repo>/saphira-cncm_b200 -lncm_b200 -lm
 */
#include <stdio.h>

static int absent(const char *what) {
    fprintf(stderr, "%s is not part of libncm_b200 (inference only): use the reference build for it\n", what);
    return 1;
}

int train_run_ex() { return absent("train"); }
int train_vq_run() { return absent("train-vq"); }
int train_qwen_run() { return absent("train-qwen"); }
int train_gpt2_run() { return absent("train-gpt2"); }
int gradcheck_run_cfg() { return absent("gradcheck"); }
int bwd_parity_run() { return absent("bwd-parity"); }
int bwdops_run() { return absent("bwdops"); }
int gpt2_cmd_taped() { return absent("gpt2-taped"); }
int qwen_cmd_taped() { return absent("qwen-taped"); }
int ckpt_info() { return absent("ckpt-info"); }
int weights_save() { absent("weights_save"); return -1; }
int vq_revive_dead() { absent("vq-revive"); return -1; }

/* live viewers: report "could not open", which the commands treat as "run without a viewer" */
int viewer_open() { return -1; }
void viewer_push() {}
int viewer_stop_requested() { return 0; }
void viewer_hold() {}
void viewer_close() {}
int viewer_active() { return 0; }
int con_viewer_open() { return -1; }
void con_viewer_push() {}
void con_viewer_close() {}
