/* CPU oracle for the DFlash speculative-verify hot path, plain C + OpenMP.
 * TEST INFRASTRUCTURE ONLY: used by the tests as a checker and by the benchmark as the timed
 * CPU baseline.  The shipped library never links or calls this file.
 *
 * Each function restates the arithmetic of the reference (paths relative to the SwiftLM
 * project root) and cites the lines it follows.  Parity of the gated-delta / replay / SDPA
 * functions is unpinned: the reference ships no golden vectors for them; see the header of
 * oracle/dflash_oracle.py for what is checked instead.
 *
 * All tensors are fp32, row-major, last axis contiguous, laid out as the reference lays them:
 *   q,k [B,T,Hk,Dk]  v,y,tape [B,T,Hv,Dv]  g [B,T,Hv] or [B,T,Hv,Dk]  beta [B,T,Hv]
 *   state [B,Hv,Dv,Dk]  mask [B,T] (step on iff > 0.5)  n [B] (step on iff t < n[b])
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Overrides the OpenMP thread count (launchers such as torchrun export OMP_NUM_THREADS=1). */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

static inline int step_on(const float* mask, const int32_t* n, int b, int t, int T) {
  /* Sources/DFlash/DFlashKernels.swift:36,115: on iff float(mask[b*T+t]) > 0.5 */
  if (mask && !(mask[(size_t)b * T + t] > 0.5f)) return 0;
  if (n && !(t < n[b])) return 0;
  return 1;
}

/* Gated-delta forward that records the innovation tape.
 * Per row of the state, in the order of Sources/DFlash/DFlashKernels.swift:440-444 (ops) and
 * :157-172 (kernel body): decay, kv = <S_row, k>, delta = (v - kv) * beta, S_row += k * delta,
 * y = <S_row, q>.  A step that is off leaves the row untouched and emits y = 0, tape = 0
 * (:446-453, :163-186).  No per-step rounding (ops semantics).  tape may be NULL. */
void oracle_gated_delta_f32(const float* q, const float* k, const float* v, const float* g,
                            const float* beta, const float* state_in, const float* mask,
                            const int32_t* n, float* y, float* state_out, float* tape,
                            int B, int T, int Hk, int Hv, int Dk, int Dv, int g_is_vector) {
  const int rep = Hv / Hk;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b) {
    for (int hv = 0; hv < Hv; ++hv) {
      const int hk = hv / rep; /* :126 */
      const float* s_in = state_in + ((size_t)b * Hv + hv) * Dv * Dk;
      float* s = state_out + ((size_t)b * Hv + hv) * Dv * Dk;
      if (s != s_in) memcpy(s, s_in, sizeof(float) * (size_t)Dv * Dk);
      for (int t = 0; t < T; ++t) {
        float* yt = y + (((size_t)b * T + t) * Hv + hv) * Dv;
        float* tp = tape ? tape + (((size_t)b * T + t) * Hv + hv) * Dv : NULL;
        if (!step_on(mask, n, b, t, T)) {
          for (int dv = 0; dv < Dv; ++dv) { yt[dv] = 0.f; if (tp) tp[dv] = 0.f; }
          continue;
        }
        const float* qt = q + (((size_t)b * T + t) * Hk + hk) * Dk;
        const float* kt = k + (((size_t)b * T + t) * Hk + hk) * Dk;
        const float* vt = v + (((size_t)b * T + t) * Hv + hv) * Dv;
        const float bt = beta[((size_t)b * T + t) * Hv + hv];
        const float* gv = g_is_vector ? g + (((size_t)b * T + t) * Hv + hv) * Dk : NULL;
        const float gs = g_is_vector ? 0.f : g[((size_t)b * T + t) * Hv + hv];
        for (int dv = 0; dv < Dv; ++dv) {
          float* row = s + (size_t)dv * Dk;
          float kv = 0.f;
          for (int i = 0; i < Dk; ++i) {
            row[i] *= gv ? gv[i] : gs;      /* :440 */
            kv += row[i] * kt[i];           /* :441 */
          }
          const float d = (vt[dv] - kv) * bt; /* :442 */
          float out = 0.f;
          for (int i = 0; i < Dk; ++i) {
            row[i] += kt[i] * d;            /* :443 */
            out += row[i] * qt[i];          /* :444 */
          }
          yt[dv] = out;
          if (tp) tp[dv] = d;
        }
      }
    }
  }
}

/* Same computation, organised the way the reference's CPU path executes it: T sequential
 * steps, each a handful of whole-state broadcast passes (decay, multiply-by-k + sum, rank-1
 * update, multiply-by-q + sum, mask blend), Sources/DFlash/DFlashKernels.swift:433-459.
 * `scratch` holds one state-sized temporary.  Used as the "reference-shaped" timed baseline. */
void oracle_gated_delta_passes_f32(const float* q, const float* k, const float* v, const float* g,
                                   const float* beta, const float* state_in, const float* mask,
                                   const int32_t* n, float* y, float* state_out, float* tape,
                                   float* scratch, int B, int T, int Hk, int Hv, int Dk, int Dv,
                                   int g_is_vector) {
  const int rep = Hv / Hk;
  const size_t rows = (size_t)B * Hv * Dv;
  if (state_out != state_in) memcpy(state_out, state_in, sizeof(float) * rows * Dk);
  float* delta = (float*)malloc(sizeof(float) * rows);
  for (int t = 0; t < T; ++t) {
    /* pass 1: decayed = state * decay (:440) */
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
      const int b = (int)(r / ((size_t)Hv * Dv)), hv = (int)((r / Dv) % Hv);
      const float* gv = g_is_vector ? g + (((size_t)b * T + t) * Hv + hv) * Dk : NULL;
      const float gs = g_is_vector ? 0.f : g[((size_t)b * T + t) * Hv + hv];
      const float* src = state_out + r * Dk;
      float* dst = scratch + r * Dk;
      for (int i = 0; i < Dk; ++i) dst[i] = src[i] * (gv ? gv[i] : gs);
    }
    /* pass 2: kv = sum(decayed * k) ; delta = (v - kv) * beta (:441-442) */
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
      const int b = (int)(r / ((size_t)Hv * Dv)), hv = (int)((r / Dv) % Hv), dv = (int)(r % Dv);
      const float* kt = k + (((size_t)b * T + t) * Hk + hv / rep) * Dk;
      const float* dst = scratch + r * Dk;
      float kv = 0.f;
      for (int i = 0; i < Dk; ++i) kv += dst[i] * kt[i];
      delta[r] = (v[(((size_t)b * T + t) * Hv + hv) * Dv + dv] - kv) * beta[((size_t)b * T + t) * Hv + hv];
    }
    /* pass 3: new = decayed + k * delta (:443) */
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
      const int b = (int)(r / ((size_t)Hv * Dv)), hv = (int)((r / Dv) % Hv);
      const float* kt = k + (((size_t)b * T + t) * Hk + hv / rep) * Dk;
      float* dst = scratch + r * Dk;
      for (int i = 0; i < Dk; ++i) dst[i] += kt[i] * delta[r];
    }
    /* pass 4: y = sum(new * q) (:444), gated outputs (:452-453) */
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
      const int b = (int)(r / ((size_t)Hv * Dv)), hv = (int)((r / Dv) % Hv), dv = (int)(r % Dv);
      const float* qt = q + (((size_t)b * T + t) * Hk + hv / rep) * Dk;
      const float* dst = scratch + r * Dk;
      float out = 0.f;
      for (int i = 0; i < Dk; ++i) out += dst[i] * qt[i];
      const float gate = step_on(mask, n, b, t, T) ? 1.f : 0.f;
      const size_t o = (((size_t)b * T + t) * Hv + hv) * Dv + dv;
      y[o] = out * gate;
      if (tape) tape[o] = delta[r] * gate;
    }
    /* pass 5: state = new * gate + state * (1 - gate) (:451) */
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
      const int b = (int)(r / ((size_t)Hv * Dv));
      if (!step_on(mask, n, b, t, T)) continue;
      memcpy(state_out + r * Dk, scratch + r * Dk, sizeof(float) * Dk);
    }
  }
  free(delta);
}

/* Tape replay: S <- S * g_t + delta_t (x) k_t, Sources/DFlash/DFlashKernels.swift:398 (ops)
 * and :64-77 (kernel body); an off step keeps the old row (:72, :402-403). */
void oracle_tape_replay_f32(const float* tape, const float* k, const float* g, const float* state_in,
                            const float* mask, const int32_t* n, float* state_out, int B, int T,
                            int Hk, int Hv, int Dk, int Dv, int g_is_vector) {
  const int rep = Hv / Hk;
#pragma omp parallel for collapse(2) schedule(static)
  for (int b = 0; b < B; ++b) {
    for (int hv = 0; hv < Hv; ++hv) {
      const int hk = hv / rep; /* :47 */
      const float* s_in = state_in + ((size_t)b * Hv + hv) * Dv * Dk;
      float* s = state_out + ((size_t)b * Hv + hv) * Dv * Dk;
      if (s != s_in) memcpy(s, s_in, sizeof(float) * (size_t)Dv * Dk);
      for (int t = 0; t < T; ++t) {
        if (!step_on(mask, n, b, t, T)) continue;
        const float* kt = k + (((size_t)b * T + t) * Hk + hk) * Dk;
        const float* tp = tape + (((size_t)b * T + t) * Hv + hv) * Dv;
        const float* gv = g_is_vector ? g + (((size_t)b * T + t) * Hv + hv) * Dk : NULL;
        const float gs = g_is_vector ? 0.f : g[((size_t)b * T + t) * Hv + hv];
        for (int dv = 0; dv < Dv; ++dv) {
          float* row = s + (size_t)dv * Dk;
          const float d = tp[dv];
          for (int i = 0; i < Dk; ++i) row[i] = row[i] * (gv ? gv[i] : gs) + kt[i] * d; /* :69 */
        }
      }
    }
  }
}

/* Block-verify SDPA, fp32.  q,out [B,Hq,16,D]; k,v [B,Hkv,N,D].
 * One key at a time with an online softmax, as the reference kernel does
 * (Sources/DFlash/DFlashKernels.swift:603-640): q pre-scaled (:593-595), running max starts
 * at the most negative finite float (:600), key n visible to row r iff n <= N_b - 16 + r (:614),
 * final divide guarded for a zero sum (:711).  kv_len may be NULL (every sequence uses N). */
void oracle_verify_sdpa_f32(const float* q, const float* k, const float* v, const int32_t* kv_len,
                            float* out, int B, int Hq, int Hkv, int N, int D, float scale) {
  const int M = 16, gqa = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic)
  for (int b = 0; b < B; ++b) {
    for (int h = 0; h < Hq; ++h) {
      const int hk = h / gqa; /* :575 */
      const int Nb = kv_len ? kv_len[b] : N;
      const float* kb = k + ((size_t)b * Hkv + hk) * N * D;
      const float* vb = v + ((size_t)b * Hkv + hk) * N * D;
      float* qs = (float*)malloc(sizeof(float) * D);
      float* o = (float*)malloc(sizeof(float) * D);
      for (int r = 0; r < M; ++r) {
        const float* qr = q + (((size_t)b * Hq + h) * M + r) * D;
        for (int i = 0; i < D; ++i) { qs[i] = scale * qr[i]; o[i] = 0.f; }
        float mx = -FLT_MAX, se = 0.f;
        const int last = Nb - M + r; /* :614 */
        for (int nn = 0; nn < Nb && nn <= last; ++nn) {
          const float* kr = kb + (size_t)nn * D;
          float sc = 0.f;
          for (int i = 0; i < D; ++i) sc += qs[i] * kr[i];
          const float nm = sc > mx ? sc : mx;
          const float f = expf(mx - nm), e = expf(sc - nm); /* :626-627 */
          mx = nm;
          se = se * f + e;
          const float* vr = vb + (size_t)nn * D;
          for (int i = 0; i < D; ++i) o[i] = o[i] * f + e * vr[i];
        }
        float* orow = out + (((size_t)b * Hq + h) * M + r) * D;
        for (int i = 0; i < D; ++i) orow[i] = se == 0.f ? o[i] : o[i] / se; /* :711 */
      }
      free(qs);
      free(o);
    }
  }
}

/* Acceptance: posterior = argmax over the vocabulary after forcing suppressed ids to -1e9
 * (Sources/DFlash/DFlashRuntime.swift:118-128; ties -> lowest index), then
 * accept = sum(cumprod(drafted[i] == posterior[i])) over i < T-1 (:133-142, :524-530).
 * logits [B,T,V]; verify_ids [B,T] (staged token then T-1 drafted); suppress [V] bytes or NULL.
 * posterior_out [B,T] uint32; accept_out [B]; next_out [B] = posterior[accept] (:547). */
void oracle_accept_f32(const float* logits, const uint8_t* suppress, const int32_t* verify_ids,
                       uint32_t* posterior_out, int32_t* accept_out, int32_t* next_out, int B, int T,
                       int V) {
#pragma omp parallel for schedule(static)
  for (int b = 0; b < B; ++b) {
    for (int t = 0; t < T; ++t) {
      const float* row = logits + ((size_t)b * T + t) * V;
      float best = 0.f;
      int arg = -1;
      for (int i = 0; i < V; ++i) {
        const float x = (suppress && suppress[i]) ? -1e9f : row[i];
        if (arg < 0 || x > best) { best = x; arg = i; }
      }
      posterior_out[(size_t)b * T + t] = (uint32_t)arg;
    }
    int acc = 0;
    for (int i = 0; i + 1 < T; ++i) {
      if ((uint32_t)verify_ids[(size_t)b * T + i + 1] != posterior_out[(size_t)b * T + i]) break;
      ++acc;
    }
    accept_out[b] = acc;
    next_out[b] = (int32_t)posterior_out[(size_t)b * T + acc];
  }
}
