/*
 * TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Persistent worker pool of the CPU checker, so that the timed CPU baseline measures the GEMV and
 * not thread start-up: the reference keeps its workers alive between calls for the same reason
 * (engine/src/cpu_mul1.rs:2114-2318). Job 0 of a batch runs on the calling thread, jobs 1..n-1 on
 * parked workers that are created once and reused; a batch returns when every job has run.
 * One batch at a time (calls from several host threads are serialised).
 */
#include <pthread.h>
#include <stdlib.h>

#define CN_POOL_MAX 256

typedef void* (*cn_job_fn)(void*);

static pthread_mutex_t g_mu = PTHREAD_MUTEX_INITIALIZER;   /* guards everything below */
static pthread_mutex_t g_batch = PTHREAD_MUTEX_INITIALIZER; /* one batch at a time */
static pthread_cond_t g_go = PTHREAD_COND_INITIALIZER, g_done = PTHREAD_COND_INITIALIZER;
static pthread_t g_thread[CN_POOL_MAX];
static int g_workers = 0;
static unsigned long g_gen = 0;
static cn_job_fn g_fn;
static char* g_jobs;
static size_t g_stride;
static int g_njobs, g_pending;

static void* worker(void* arg) {
    const int me = (int)(long)arg; /* worker i runs job i + 1 of every batch that has one */
    unsigned long seen = 0;
    pthread_mutex_lock(&g_mu);
    for (;;) {
        while (g_gen == seen) pthread_cond_wait(&g_go, &g_mu);
        seen = g_gen;
        if (me + 1 < g_njobs) {
            cn_job_fn fn = g_fn;
            void* job = g_jobs + (size_t)(me + 1) * g_stride;
            pthread_mutex_unlock(&g_mu);
            fn(job);
            pthread_mutex_lock(&g_mu);
            if (--g_pending == 0) pthread_cond_signal(&g_done);
        }
    }
    return NULL;
}

/* run fn(jobs + i * stride) for i in 0..n-1, job 0 on the caller */
void cn_o_pool_run(cn_job_fn fn, void* jobs, size_t stride, int n) {
    if (n <= 1) {
        if (n == 1) fn(jobs);
        return;
    }
    if (n > CN_POOL_MAX + 1) n = CN_POOL_MAX + 1; /* callers never ask for more; jobs beyond would be lost */
    pthread_mutex_lock(&g_batch);
    pthread_mutex_lock(&g_mu);
    while (g_workers < n - 1) {
        if (pthread_create(&g_thread[g_workers], NULL, worker, (void*)(long)g_workers) != 0) abort();
        pthread_detach(g_thread[g_workers]);
        g_workers++;
    }
    g_fn = fn, g_jobs = (char*)jobs, g_stride = stride, g_njobs = n, g_pending = n - 1;
    g_gen++;
    pthread_cond_broadcast(&g_go);
    pthread_mutex_unlock(&g_mu);
    fn(jobs);
    pthread_mutex_lock(&g_mu);
    while (g_pending > 0) pthread_cond_wait(&g_done, &g_mu);
    g_njobs = 0;
    pthread_mutex_unlock(&g_mu);
    pthread_mutex_unlock(&g_batch);
}
